from .engine import ServingEngine  # noqa: F401
from .kv_cache import PageAllocator, PagedKVCache  # noqa: F401
from .scheduler import Request, Scheduler, poisson_trace  # noqa: F401
from .server import Completion, EngineServer, QueueFull, build_app  # noqa: F401
