"""Architectures.  Importing the package registers them; another architecture is one
more module here: a typed configuration, a function from it to a `ModelSpec`, and a
`register_architecture` call."""
from . import lfm2  # noqa: F401
