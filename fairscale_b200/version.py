__version_tuple__ = (0, 1, 0)
