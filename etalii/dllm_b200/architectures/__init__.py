from . import llama, tisalorn  # noqa: F401  (register the architectures)
