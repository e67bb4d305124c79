"""Typed errors of the configuration layer."""


class ConfigError(ValueError):
    """A config.json or recipe key is missing, ill-typed or asks for something
    the engine refuses.  The message names the key."""
