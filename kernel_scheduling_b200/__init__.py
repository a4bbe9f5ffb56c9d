"""B200-native trace -> interference-table pipeline (drop-in for the reference's offline post-processing)."""
__version__ = "0.1.0"
