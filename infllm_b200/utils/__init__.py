"""Callers' side of the attention-forward API: model patching and a chunked greedy driver
(inf_llm/utils/patch.py, inf_llm/utils/greedy_search.py)."""
from .decoder import HeadGroupDecoder
from .greedy_search import GreedySearch
from .patch import patch_hf

__all__ = ["patch_hf", "GreedySearch", "HeadGroupDecoder"]
