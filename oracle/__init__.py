"""CPU oracle for the extraction + split SpMV path.  TEST INFRASTRUCTURE ONLY: nothing in the shipped package may
import this; only tests/, the smoke check and the CPU-baseline leg of bench.py do."""
from .oracle import *  # noqa: F401,F403
