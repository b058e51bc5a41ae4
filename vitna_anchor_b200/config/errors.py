"""What every architecture's configuration reader and the registry raise."""


class ConfigError(ValueError):
    """config.json is missing, malformed, names no registered architecture, or asks for what the engine lacks."""
