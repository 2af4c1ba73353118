"""Process-wide device context (reference: flash3dxfmr/psh/dev_context.py:9-34)."""
from __future__ import annotations

from ..lib import pshattn

DEV_MGR = pshattn.DeviceManagerSingleton.instance()
ENABLE_NVTX = False


def get_dev_manager():
    return DEV_MGR


def init_dev(dev_id: int):
    assert isinstance(dev_id, int), f"Expect dev_id is an int, got {type(dev_id)}"
    DEV_MGR.init_dev_info(dev_id)


def get_sync_stream():
    return DEV_MGR.get_sync_stream()


def set_sync_stream(is_syncing: bool):
    return DEV_MGR.set_sync_stream(is_syncing)


def set_nvtx(flag: bool):
    # the reference assigns a function-local here (dev_context.py:30-31), so NVTX can never be switched on
    # through its API; this build sets the module flag
    global ENABLE_NVTX
    ENABLE_NVTX = bool(flag)


def get_nvtx():
    return ENABLE_NVTX
