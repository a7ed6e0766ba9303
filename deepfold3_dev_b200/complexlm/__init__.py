"""Masked language model over protein complexes (side model; reference: complexlm/).

Chain-scoped rotary attention layers alternate with complex-scoped layers that carry no positions, over one packed token
axis. ``config`` holds the experiment description, ``model`` the network and the packed batch, ``data`` the flat store,
sampling, cropping, masking and packing, ``trainer`` the training loop, ``prepare`` the store builders.
"""

from .config import ComplexLMConfig, ExperimentConfig, load_experiment  # noqa: F401
from .model import ComplexLM, PackedBatch  # noqa: F401
