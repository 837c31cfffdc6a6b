"""Import-path compatibility with the reference package layout (``wall_x.*``).

Everything here re-exports :mod:`wallx_b200`; no code lives in this package.
"""
