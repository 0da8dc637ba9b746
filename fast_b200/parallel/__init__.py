from .comm import Communicator, LocalGroup, Schedule  # noqa: F401
