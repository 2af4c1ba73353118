"""B200-native kernels and host-side mirror of the Flash3D data-parallel hot path.

Sub-packages: `lib` (shared library + operator module `pshattn`), `psh` (host buffer planning), `layers` (the
nn.Module tree of the Flash3D backbone), `synthetic` (seeded stand-ins for the benchmark point clouds).
"""
