from . import llama, satavik, tisalorn  # noqa: F401  (register the architectures)
