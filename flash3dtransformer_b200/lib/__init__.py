"""Native library and its operator module (ctypes mirror of the reference's `flash3dxfmr.lib.pshattn`)."""
