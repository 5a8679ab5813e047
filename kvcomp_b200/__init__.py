"""kvcomp_b200: the KV-cache compression hot path of BoJiang03/kvcomp, rebuilt for B200 (sm_100a).

    kvcomp_b200.ops          torch-facing wrappers over the C ABI (include/kvcomp_b200.h)
    kvcomp_b200.kvcomp_cuda  the reference's operator module, same names and arguments
    kvcomp_b200.cache        KVCompCtx / KVCompCache, the reference's cache classes
    kvcomp_b200.synth        seeded synthetic K/V with the benchmark's distributions

Everything computes on the GPU through libkvcomp_b200.so; there is no CPU fallback.
"""
__version__ = "0.1.0"
