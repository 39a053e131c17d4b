"""B200-native prefill->decode KV handoff for vllm-rlt.

Importing this package loads no native code and creates no CUDA context; the
C-ABI library is loaded on first use (``vllm_rlt_b200._lib.load``).
"""

__version__ = "0.1.0"
