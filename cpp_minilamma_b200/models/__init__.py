"""Architectures.  Importing the package registers them by their `architectures` name."""
from . import badolix, kupirax, llama, malulorn, sopanex  # noqa: F401
