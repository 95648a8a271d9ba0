from .comm import Communicator, SingleProcessComm, TorchDistComm, make_communicator  # noqa: F401
from .ddp import DDP, GradBucket  # noqa: F401
from .fsdp import FSDP, FSDPUnit  # noqa: F401
