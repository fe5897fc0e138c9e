"""Kernels. ``cuda`` holds the compiled sm_100a kernels, ``reference`` their plain PyTorch statements."""
