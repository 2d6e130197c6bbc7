"""The step function, the engine around it and the scheduler above it."""
from .engine import BlockManager, CapacityError, Engine
from .scheduler import ContinuousBatchScheduler

__all__ = ["BlockManager", "CapacityError", "Engine", "ContinuousBatchScheduler"]
