from .experts import GroupedExperts  # noqa: F401
from .moe_layer import MOELayer  # noqa: F401
from .top2gate import Top2Gate, Top2Route, top2_route, top2gating  # noqa: F401
