"""Parts a layer is made of: mixer, feed-forward, norm, position encoding, block."""
from . import registry, spec  # noqa: F401
