from enum import Enum


class ExitCode(Enum):
    """Process exit codes of the ``wgit`` command."""

    CLEAN = 0
    FILE_EXISTS_ERROR = 1
    FILE_DOES_NOT_EXIST_ERROR = 2
    ERROR = 3
