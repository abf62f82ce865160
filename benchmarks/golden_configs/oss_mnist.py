"""Regression bars of the OSS / ShardedDDP benchmark (reference: benchmarks/golden_configs/oss_mnist.py:7-18)."""


def get_golden_real_stats():
    return {"reference_speed": 578, "reference_memory": 640, "reference_loss": 0.026}


def get_golden_synthetic_stats():
    raise NotImplementedError("Synthetic data benchmarks are not supported.")
