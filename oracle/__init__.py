"""TEST INFRASTRUCTURE ONLY: CPU restatements of the reference's algorithms, used as the checker.

Nothing under this folder is product code; only tests/, __graft_entry__.smoke() and the
CPU-baseline legs of bench.py may import it.
"""
