"""B200-native permutohedral-lattice filter: hand-written sm_100a CUDA kernels behind a C ABI
(include/pl_lattice.h), with a host-side mirror of the reference operator."""
from .lattice_filter import (compute_positions, export_lattice, filter_positions, lattice_filter,  # noqa: F401
                             lattice_filter_raw, lattice_stats, release_workspaces, check_pending, Lattice)
from .host_pipeline import HostPipeline  # noqa: F401,E402
from .graphed import GraphedLatticeFilter  # noqa: F401,E402
from .crf import DenseCRF  # noqa: F401,E402
from .capi import PlError  # noqa: F401,E402
from .sharding import OutputGather, lattice_filter_sharded, shard_range  # noqa: F401,E402
