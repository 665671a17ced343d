"""Fused-kernel generator: emits one persistent, warp-specialised kernel per (tzgemm, CUDA-core) pair and
thread ratio, compiles it into a loadable module and smoke-tests it (the B200 form of the reference's
fusion/code/gen_run.py, gen_mix.py, data.py, gen_test.py)."""
