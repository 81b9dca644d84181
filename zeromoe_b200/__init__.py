"""zeromoe_b200 -- B200 (sm_100a) implementation of ZeroMoE's MoE expert hot
path behind its operator surface.  The product is libzmoe_b200.so (C ABI in
include/zmoe_b200.h); this package is the thin Python binding used by the tests
and the benchmark.  There is no CPU fallback: importing `zeromoe_b200.lib`
without the built library raises.
"""
__all__ = ["lib", "synth", "build"]
