"""tuff_b200: a single-GPU inference engine for NVIDIA B200 (sm_100a), built
from parts, for the LFM2 / LFM2.5 dense decoder."""
__version__ = "0.1.0"
