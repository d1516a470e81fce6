from .loader import load_model, route_checkpoint_name  # noqa: F401
