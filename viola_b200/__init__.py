"""viola_b200: a Blackwell-datacenter (B200, sm_100a) native FP8 training framework."""

__version__ = "0.1.0"
