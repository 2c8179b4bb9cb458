"""CUDA sources (sm_100a) and their build."""
