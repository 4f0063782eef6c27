"""Built-in architectures.  Importing this package registers them."""

from emberserve_b200.models import qwen2  # noqa: F401
