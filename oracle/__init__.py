"""CPU oracle for the SNN-TC operators -- TEST INFRASTRUCTURE ONLY (never imported by the product)."""
from .oracle import *  # noqa: F401,F403
