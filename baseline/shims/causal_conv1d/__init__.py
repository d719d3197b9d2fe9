"""Import-time stand-in for the `causal_conv1d` package (see causal_conv1d_cuda.py in this folder)."""
