"""Expert-parallel all-to-all kernels (dispatch / combine) and their baselines."""
