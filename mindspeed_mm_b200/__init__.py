"""B200-native multimodal training framework with the capabilities of MindSpeed-MM."""
__version__ = "0.1.0"
