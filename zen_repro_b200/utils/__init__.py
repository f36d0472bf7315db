from .logging import setup_logger  # noqa: F401
from .seed import set_seed  # noqa: F401
from .trace import trace_range, enable_tracing  # noqa: F401
