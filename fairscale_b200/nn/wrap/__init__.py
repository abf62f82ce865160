from .auto_wrap import (  # noqa: F401
    ConfigAutoWrap,
    auto_wrap,
    config_auto_wrap_policy,
    default_auto_wrap_policy,
    enable_wrap,
    wrap,
)
