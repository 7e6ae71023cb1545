"""infllm_b200 — InfLLM's per-layer context-memory attention on B200 (sm_100a).

Drop-in for the reference's attention-forward API: `infllm_b200.attention` mirrors
`inf_llm.attention` (RotaryEmbeddingESM, ATTN_FORWRAD["inf-llm"], ContextManager, the multi-stage
attention class).  All compute runs in libinfllm_b200.so (CUDA, C ABI in include/infllm_b200.h)."""
__version__ = "0.1"
