"""Error types raised while reading a model folder."""


class ConfigError(ValueError):
    """config.json is missing a key, holds a wrong type, or names sizes that do not fit together."""


class UnknownArchitectureError(ConfigError):
    """config.json names an architecture nobody registered."""
