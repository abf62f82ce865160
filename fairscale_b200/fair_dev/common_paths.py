"""Common cache root for datasets downloaded by benchmark and test helpers."""
DATASET_CACHE_ROOT = "cached_datasets"
