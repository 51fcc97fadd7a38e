"""Hand-written sm_100a operators and the nn modules built on them."""
from .backend import set_backend, get_backend  # noqa: F401
