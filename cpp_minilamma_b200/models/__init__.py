"""Architectures.  Importing the package registers them by their `architectures` name."""
from . import kupirax, llama, malulorn, sopanex  # noqa: F401
