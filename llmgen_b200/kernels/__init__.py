"""CUDA kernels for sm_100a: build driver (`build`) and bindings (`ops`)."""
