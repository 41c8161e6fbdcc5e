from .exception import ParametersInvalid, ConfigError, ModelInitError, ModelExecError, logger

__all__ = ["ParametersInvalid", "ConfigError", "ModelInitError", "ModelExecError", "logger"]
