from .env import knobs, Knobs  # noqa: F401
