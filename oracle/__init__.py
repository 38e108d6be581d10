"""CPU oracle for the FlashMoE forward path.

TEST INFRASTRUCTURE ONLY.  Nothing in the product package imports this; it is
used by the tests, by the smoke check and by the CPU-baseline legs of the
benchmark as the checker / timed CPU arm, never as a compute path of the
library.
"""
