"""The kernels' status word as seen from the layer API.

Every bounded wait inside a kernel that runs out makes its thread block unwind, fill its output rows
with NaN and set a per-device status word; while the word is set, later launches of those kernels leave
at once and mark their rows too.  Reading the word synchronises the device, so the layer API does it
only where it synchronises anyway (the host-operand entry points) or when asked to:

    MINDIESD_CHECK_STATUS=1   attention_forward, sparse_attention, attention_forward_varlen and
                              FP8RotateQuantFA read the word after every call and raise ModelExecError
"""
import os

from .exception import ModelExecError


def check_enabled() -> bool:
    return os.environ.get("MINDIESD_CHECK_STATUS", "0") not in ("", "0", "false", "False")


def raise_if_kernel_gave_up(where: str) -> None:
    """Synchronises the current device, reads (and clears) its status word, raises if it was set."""
    from .. import _cabi
    code = _cabi.device_status()
    if code != 0:
        raise ModelExecError(f"{where}: a kernel gave up a bounded wait (device status {code}); the outputs of this "
                             "and of every call since are filled with NaN and must be recomputed.")


def checked(result, where: str):
    """`result` unchanged; with MINDIESD_CHECK_STATUS=1 the status word is read first."""
    if check_enabled():
        raise_if_kernel_gave_up(where)
    return result
