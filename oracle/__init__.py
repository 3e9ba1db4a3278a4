"""CPU oracle for the vortx matmul path — TEST INFRASTRUCTURE ONLY.

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline / reference arm may import
this package.  It is the checker, never the thing shipped or measured as the product.
"""
from .oracle import *  # noqa: F401,F403
