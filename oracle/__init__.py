"""TEST INFRASTRUCTURE ONLY: CPU restatements the CUDA kernels are checked against.

Only tests/, __graft_entry__.smoke() and bench.py's cpu_baseline / reference legs may
import this package; nothing under kohaku_tt_b200/ does.
"""
