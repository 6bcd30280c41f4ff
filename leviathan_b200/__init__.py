"""B200-native quantized-weight hot path of Leviathan (Q4_0 / Q4_K / Q6_K
dequant-fused matvec, prefill dequant-GEMM, routed MoE) behind the C ABI of
libleviathan_cuda.so.  Importing the package does not load the library;
creating a Context does, and fails loudly if it is not built."""
from ._lib import (GGML_Q4_0, GGML_Q4_K, GGML_Q6_K, SCHEDULE_AUTO, SCHEDULE_PLAIN,  # noqa: F401
                   SCHEDULE_STREAM, LIB_PATH)
from .api import Context, GGUFFile, LevError, MoEWeights, PagedKV, Weights  # noqa: F401

__all__ = ["Context", "LevError", "Weights", "MoEWeights", "GGUFFile", "PagedKV", "GGML_Q4_0", "GGML_Q4_K", "GGML_Q6_K",
           "SCHEDULE_AUTO", "SCHEDULE_PLAIN", "SCHEDULE_STREAM", "LIB_PATH"]
