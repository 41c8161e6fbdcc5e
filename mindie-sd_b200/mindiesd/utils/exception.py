"""Exception types of the layer API.  Callers of MindIE-SD catch these by name, and the message
prefix carries the error code (mindiesd/utils/exception.py:16-48 of MindIE-SD)."""
import logging

logger = logging.getLogger("mindiesd")


class _CodedError(Exception):
    code = "MIE06E000000"

    def __init__(self, message=""):
        self.message = f"[{self.code}] {message}"
        logger.error(self.message)
        super().__init__(self.message)


class ParametersInvalid(_CodedError):
    code = "MIE06E000001"


class ConfigError(_CodedError):
    code = "MIE06E000002"


class ModelInitError(_CodedError):
    code = "MIE06E000003"


class ModelExecError(_CodedError):
    code = "MIE06E000004"


class TimeoutError(_CodedError):  # noqa: A001 - the reference exports this name
    code = "MIE06E000005"
