"""Native kernels: build, load and tensor-level wrappers."""
