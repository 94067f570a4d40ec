"""Architectures.  Importing this package registers them."""
from . import llama  # noqa: F401
from . import gekavik  # noqa: F401
from . import medirax  # noqa: F401
from . import sorupel  # noqa: F401
from . import kafepel  # noqa: F401
