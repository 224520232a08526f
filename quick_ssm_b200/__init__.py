"""B200-native gated linear scan with the interface of quick_ssm (reference: quick_ssm/__init__.py:1-4)."""
from .scan_interface import scan
from .layers import SSM, RMSNorm

__all__ = ["scan", "SSM", "RMSNorm"]
