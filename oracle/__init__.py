"""CPU restatement of the reference's affix-KV-reuse path.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package imports this; it is
the checker that the CUDA path is compared against (tests, the smoke check and
the CPU-baseline leg of the benchmark).  Every function cites the reference
lines it restates.  The restatement itself is pinned against the reference's
own code (imported in the build container) by the fixtures under
``tests/golden`` and the script that generated them.
"""
