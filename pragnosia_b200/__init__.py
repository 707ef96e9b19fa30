"""B200-native carrier kernels behind the reference's Python operator API.

Importing the package does not load the CUDA library; the first op call does, and raises if it is missing.
"""
__version__ = "0.1.0"
