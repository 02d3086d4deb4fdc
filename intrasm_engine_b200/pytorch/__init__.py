"""PyTorch-facing layer: operators, autograd functions, graph constructor, CSR helpers."""
