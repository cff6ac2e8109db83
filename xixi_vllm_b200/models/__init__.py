"""Model definitions, tensor-parallel layers and weight loading."""
