"""linear_moe_b200 — a Blackwell-native (sm_100a) Linear-MoE training framework."""
__version__ = "0.1.0"
