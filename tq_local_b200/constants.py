"""Defaults shared by the generation entry points."""

# Cap on new tokens used by ``TurboQuantSession.generate`` (same value as the reference's
# ``src/turboquant/constants.py``).
DEFAULT_MAX_NEW_TOKENS = 1024
