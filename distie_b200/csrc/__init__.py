"""Native sources (CUDA kernels for sm_100a, the C++ block pool) and their builder."""
