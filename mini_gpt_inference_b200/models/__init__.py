from . import minigpt  # noqa: F401  (registers the architecture)
