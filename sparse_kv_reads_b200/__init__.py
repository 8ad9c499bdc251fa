"""B200-native clustered sparse KV-cache decode attention (CUDA kernels behind a C ABI)."""

from .accounting import kv_read_fraction, overhead_rows, step_bytes  # noqa: F401
from .cluster_state import ClusterArena, SphereIndexFused, SphereIndexGraph  # noqa: F401
from .graph_decode import AllLayerInsert, DenseAttentionGraph, GraphDecoder  # noqa: F401
from .patch import ReadStats, install, make_decode_op, uninstall  # noqa: F401
from .qwen3 import Qwen3Config, Qwen3Model, apply_rope  # noqa: F401
