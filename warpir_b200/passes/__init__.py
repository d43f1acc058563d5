"""Scheduling passes retargeted to the sm_100a machine model."""
