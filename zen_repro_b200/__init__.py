"""B200-native sparse gradient synchronisation framework (ZEN capabilities, sm_100a kernels)."""
__version__ = "0.1.0"
