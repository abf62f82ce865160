"""`install_as_fairscale()`: reference import paths and reference pickles resolve to this package."""
import pickle
import sys

import pytest
import torch
from torch import nn

from fairscale_b200 import compat


def test_alias_imports_and_unpickles_reference_class_paths():
    assert "fairscale" not in sys.modules
    compat.install_as_fairscale()
    try:
        compat.install_as_fairscale()  # idempotent
        import fairscale  # noqa: F401
        from fairscale.nn import FullyShardedDataParallel, checkpoint_wrapper  # noqa: F401
        from fairscale.nn.misc.flatten_params_wrapper import FlatParameter
        from fairscale.optim import OSS  # noqa: F401
        import fairscale.experimental.nn.offload as off

        import fairscale_b200
        from fairscale_b200.nn.misc.flatten_params_wrapper import FlatParameter as Ours

        assert fairscale is fairscale_b200 and FlatParameter is Ours
        assert off is sys.modules["fairscale_b200.experimental.nn.offload"]
        # a pickle that names the class by the reference's module path
        flat = Ours([nn.Parameter(torch.ones(2, 2)), nn.Parameter(torch.zeros(3))])
        # protocol 2 writes class references as newline-terminated text (no length prefix), so the path can be swapped
        blob = pickle.dumps(flat, protocol=2).replace(b"fairscale_b200.nn.misc", b"fairscale.nn.misc")
        assert b"fairscale.nn.misc.flatten_params_wrapper" in blob
        back = pickle.loads(blob)
        assert isinstance(back, Ours) and back.numel() == 7 and [tuple(v.shape) for v in back.get_param_views()] == [(2, 2), (3,)]
        with pytest.raises(ImportError):
            import fairscale.does_not_exist  # noqa: F401
    finally:
        compat.uninstall()
    assert "fairscale" not in sys.modules and "fairscale.nn" not in sys.modules
    with pytest.raises(ImportError):
        import fairscale  # noqa: F401,F811
