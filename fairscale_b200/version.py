__version__ = "0.1.0"
# API level of facebookresearch/fairscale that this library mirrors (fairscale/version.py:1).
FAIRSCALE_API_VERSION = "0.4.13"
