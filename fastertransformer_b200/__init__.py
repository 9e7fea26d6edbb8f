"""B200-native (sm_100a) implementation of FasterTransformer's per-step decode sampling path.

The product is the C-ABI shared library declared in include/ftb200.h (built in-tree by
`python -m fastertransformer_b200.build`).  This package loads it through ctypes and offers a thin
host-side mirror of the reference's layer interface for tests and benchmarks.  Touching any kernel
entry point without the built library raises ImportError: there is no CPU fallback.
"""

_LAZY = {
    "lib": "._lib", "FtbError": "._lib", "SamplingParams": "._lib", "check": "._lib",
    "BeamParams": "._lib", "BeamHyps": "._lib", "GatherTreeParams": "._lib",
    "DynamicDecodeLayer": ".decode_layer", "DynamicDecodeOp": ".th_decode_op",
    "VocabParallelSampler": ".vocab_parallel", "log_prob_from_logits": ".logprob",
}


def __getattr__(name):
    # resolved on first use so that `python -m fastertransformer_b200.build` can run before the
    # library exists; everything else fails loudly if it is missing
    if name in _LAZY:
        import importlib
        return getattr(importlib.import_module(_LAZY[name], __name__), name)
    raise AttributeError(name)
