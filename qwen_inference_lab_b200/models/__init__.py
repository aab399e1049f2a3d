"""Importing this package registers every architecture the engine knows."""
from . import qwen3  # noqa: F401
from . import virulix  # noqa: F401
from . import debisun  # noqa: F401
from . import larolorn  # noqa: F401
from . import gogotar  # noqa: F401
