"""B200-native vision-language-action training and inference framework."""
__version__ = "0.1.0"
