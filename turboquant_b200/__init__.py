"""B200-native TurboQuant KV-cache hot paths (cache write + paged decode attention)."""
__version__ = "0.1.0"
