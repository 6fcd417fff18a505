"""The hand-written CUDA kernels (sm_100a) and their Python surface."""
