class ConfigError(ValueError):
    """A config.json key is missing, has the wrong type, or asks for what the engine does not build."""
