"""Built-in architectures: importing this package registers them."""
from . import gemma, pesanex, taritar  # noqa: F401
