from .launch import launch_from_torch  # noqa: F401
from .mesh import ProcessGroupMesh  # noqa: F401
from .coordinator import DistCoordinator  # noqa: F401
from .reducer import ZenDDP, GradBucket  # noqa: F401
from .hooks import compress, compress_with_allgather, make_zen_comm_hook  # noqa: F401
from .plugin import Booster, HybridParallelPlugin  # noqa: F401
from .embedding_sync import EmbeddingRowSync  # noqa: F401
from .failure import Heartbeat, PeerLost  # noqa: F401
