"""B200-native compute/communication overlap kernel library (work in progress)."""
__version__ = "0.1.0"
