"""CUDA sources for sm_100a and the builder that compiles and loads them."""
