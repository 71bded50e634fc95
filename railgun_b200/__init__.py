"""railgun_b200: a small inference engine for one B200, after Atari-Katana/railgun."""
__version__ = "0.1.0"
