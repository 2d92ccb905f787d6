"""CUDA sources for sm_100a, their build script and their Python face."""
