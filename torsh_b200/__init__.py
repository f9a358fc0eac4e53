"""torsh_b200: a Blackwell-native deep-learning framework with ToRSh's API shape."""
__version__ = "0.1.0"
