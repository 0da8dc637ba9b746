from .comm import Communicator, LocalGroup, Schedule  # noqa: F401
from .p2p_executor import P2PExecutor  # noqa: F401
from .autograd import all_to_all_v  # noqa: F401
