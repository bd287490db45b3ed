"""B200-native NEO-unify (SenseNova-U1) training and inference framework."""
__version__ = "0.1.0"
