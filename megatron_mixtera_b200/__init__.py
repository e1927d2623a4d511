"""B200-native decode step for Megatron Core dynamic inference (host side + sm_100a kernels)."""
__version__ = "0.1.0"
