"""CPU checkers for the speculative-decoding path (TEST INFRASTRUCTURE, never product code).

carat_semantics.py  torch-CPU restatement of the reference's verify / draft numerics and bookkeeping
accept.c            plain-C restatement of the integer logic (built by oracle/Makefile)
ref_speculation_shim.cpp + Makefile `ref` target: the reference's own speculation.cpp compiled
                    unmodified into oracle/_ref/ where the reference tree is present

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline legs may import or load anything
under this directory.
"""
