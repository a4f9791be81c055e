"""Architectures.  Importing this package registers them."""
from . import qwen2  # noqa: F401
from . import kunonex  # noqa: F401
from . import pemorax  # noqa: F401
from . import tekosun  # noqa: F401
from . import malazen  # noqa: F401
