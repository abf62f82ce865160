from .dynamic_loss_scaler import DynamicLossScaler  # noqa: F401

__all__ = ["DynamicLossScaler"]
