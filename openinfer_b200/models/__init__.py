"""Built-in architectures. Importing this package registers them."""
from . import bubalix, delunex, luzitar, pilonex, qwen3  # noqa: F401
