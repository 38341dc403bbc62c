"""Built-in architectures.  Importing this package registers them."""
from . import malapel, qwen3, sakinex, sarizen, ziginex  # noqa: F401
