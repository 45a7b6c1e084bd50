from .model import Layer, Model, declared_tensors, load_model, resolve_dtype

__all__ = ["Layer", "Model", "declared_tensors", "load_model", "resolve_dtype"]
