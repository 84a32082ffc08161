"""fastmace_b200: a B200-native (sm_100a) MACE energy / forces / stress engine behind FastMACE's force-field boundary."""

__version__ = "0.1.0"
