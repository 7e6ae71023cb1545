"""Import the Python reference (thunlp/InfLLM) on a machine without a GPU.

Used by make_golden.py, on a machine that has the reference checkout (the
fixtures it writes are what travels), and by the reference arm of bench.py
(`--impl reference`), which times the reference's own ContextManager on the
host cores from an unmodified copy of its package.  Nothing under the package
and none of the GPU tests imports this file.

The reference hard-codes CUDA in a few places (inf_llm/attention/rope.py:23,
inf_llm/attention/context_manager.py:13,122,133,306) and calls
torch.cuda.Event / Stream / current_stream / stream.  The hook below rewrites
those device literals to "cpu" at import time (source on disk is untouched) and
stubs the stream API with no-ops, so the reference's own arithmetic runs
unchanged on the host.
"""
import contextlib
import importlib.abc
import importlib.machinery
import os
import sys

import torch

_REWRITES = (
    ('device="cuda"', 'device="cpu"'),
    ("device='cuda'", "device='cpu'"),
    ('device = "cuda"', 'device = "cpu"'),
    ("assert _t.is_cuda", "pass"),
)


class _Loader(importlib.machinery.SourceFileLoader):
    def get_data(self, path):
        data = super().get_data(path)
        if path.endswith(".py"):
            text = data.decode("utf-8")
            for a, b in _REWRITES:
                text = text.replace(a, b)
            data = text.encode("utf-8")
        return data

    def get_code(self, fullname):
        # compile from the rewritten source; never touch __pycache__
        path = self.get_filename(fullname)
        return compile(self.get_data(path), path, "exec", dont_inherit=True)


class _Finder(importlib.abc.MetaPathFinder):
    def __init__(self, root):
        self.root = root

    def find_spec(self, fullname, path=None, target=None):
        if fullname != "inf_llm" and not fullname.startswith("inf_llm."):
            return None
        rel = fullname.replace(".", os.sep)
        pkg = os.path.join(self.root, rel, "__init__.py")
        mod = os.path.join(self.root, rel + ".py")
        if os.path.exists(pkg):
            return importlib.machinery.ModuleSpec(
                fullname, _Loader(fullname, pkg), origin=pkg, is_package=True
            )
        if os.path.exists(mod):
            return importlib.machinery.ModuleSpec(fullname, _Loader(fullname, mod), origin=mod)
        return None


class _Event:
    def __init__(self, *a, **k):
        pass

    def record(self, *a, **k):
        pass

    def wait(self, *a, **k):
        pass

    def synchronize(self):
        pass


class _Stream:
    def __init__(self, *a, **k):
        pass

    def wait_stream(self, *a, **k):
        pass


def install(root):
    """Make `import inf_llm.attention...` resolve to the CPU-rewritten reference."""
    if not os.path.isdir(os.path.join(root, "inf_llm")):
        raise FileNotFoundError(f"reference checkout not found at {root}")
    if not any(isinstance(f, _Finder) for f in sys.meta_path):
        sys.meta_path.insert(0, _Finder(root))
    torch.cuda.Event = _Event
    torch.cuda.Stream = _Stream
    torch.cuda.current_stream = lambda *a, **k: _Stream()
    torch.cuda.stream = lambda *a, **k: contextlib.nullcontext()
    torch.Tensor.pin_memory = lambda self, *a, **k: self
    # import only the modules of the path; inf_llm/__init__ pulls in transformers patches
    import types

    if "inf_llm" not in sys.modules:
        pkg = types.ModuleType("inf_llm")
        pkg.__path__ = [os.path.join(root, "inf_llm")]
        sys.modules["inf_llm"] = pkg
    import inf_llm.attention.context_manager as cm  # noqa: E402
    import inf_llm.attention.rope as rope  # noqa: E402
    from inf_llm.attention.dot_production_attention.torch_impl import (  # noqa: E402
        TorchMultiStageDotProductionAttention,
    )

    return cm, rope, TorchMultiStageDotProductionAttention
