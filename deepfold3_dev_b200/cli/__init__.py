"""Command line entry points (``python -m deepfold3_dev_b200.cli``)."""

from .main import cli, main  # noqa: F401
