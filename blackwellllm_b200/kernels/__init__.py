"""Hand-written CUDA kernels for sm_100a (sources in ``csrc/``) and their Python face."""
