"""Model zoo.  Sub-packages are imported lazily by dotted path from configs."""
from . import convert_weights  # noqa: F401
