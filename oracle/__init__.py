"""CPU restatement of the reference hot path — TEST INFRASTRUCTURE ONLY.

Only tests/, __graft_entry__.smoke() and bench.py's cpu_baseline / --impl reference legs may
import this package, and only as the checker or the timed CPU baseline.  Nothing in
mdlarc_scale_b200/ imports it.

Parity status: PINNED.  tests/golden/ holds outputs of the reference implementation itself
(imported from its source tree by tests/golden/make_golden.py): fp32 logits, greedy tokens,
3D positions, dihedral/colour-permutation results and AAIVR votes on seeded inputs, plus the
known-answer values of the reference's own tests; tests/test_oracle_golden.py checks every
function here against them.
"""
