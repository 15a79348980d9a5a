"""Python side of the hand-written sm_100a kernels: build, load, and tensor-level wrappers."""
