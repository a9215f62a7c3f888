"""Built-in architectures.  Importing this package registers them."""
from . import qwen2  # noqa: F401
