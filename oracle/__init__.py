"""Parity checker (test infrastructure). Only tests/, the smoke check and the bench's CPU-baseline
leg import this package; nothing under luma_b200/ does."""
