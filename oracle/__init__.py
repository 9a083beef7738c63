"""CPU oracle package: test infrastructure only (checker and timed CPU baseline).

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline legs may import it.
"""
