from .pyconfig import initialize, HyperParameters, ConfigError  # noqa: F401
