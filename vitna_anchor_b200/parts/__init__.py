from .base import Block, FeedForward, GroupMeta, Mixer, Norm, Part, PositionEncoding, StepContext, Workspace  # noqa: F401
from .registry import make_part, register_part  # noqa: F401
