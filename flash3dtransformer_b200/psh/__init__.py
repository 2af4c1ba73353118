"""Host-side buffer planning for the PSH operators (mirror of the reference's flash3dxfmr/psh package)."""
