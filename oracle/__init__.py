"""CPU restatement of the reference's arithmetic for the hot path.  TEST INFRASTRUCTURE ONLY.

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline / reference arm may import
this package, and only as the checker or the timed CPU baseline -- never as a product path.
"""
