from . import attention, block, norm, position, shortconv, swiglu  # noqa: F401  (registers the parts)
from .base import PagedView, PositionArgs, SlotView, StepContext, Workspace
from .registry import build, register, registered
