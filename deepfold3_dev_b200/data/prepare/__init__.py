"""Dataset preparation: mmCIF -> filtered structures, sequence clusters, manifest, packs (reference: data/prepare/)."""

from .filters import StructureFilterConfig, filter_structure, filter_structure_metadata, select_interface_chains  # noqa: F401
from .clustering import cluster_records  # noqa: F401
from .pipeline import prepare_directory, process_entry  # noqa: F401
