from .gossip import SlowMoBaseAlgorithm, SlowMoDistributedDataParallel  # noqa: F401

__all__ = ["SlowMoBaseAlgorithm", "SlowMoDistributedDataParallel"]
