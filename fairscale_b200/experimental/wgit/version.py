__version_tuple__ = (0, 0, 1)
