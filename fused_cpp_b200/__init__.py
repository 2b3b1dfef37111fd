"""B200-native routed-expert MoE path behind the fused_cpp operator API."""
__version__ = "0.1.0"
