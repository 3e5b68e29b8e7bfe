"""kernel_align_b200: a Blackwell-native (sm_100a) RL post-training operator library."""

__version__ = "0.1.0"
