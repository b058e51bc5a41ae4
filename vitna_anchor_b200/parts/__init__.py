from .base import (Block, FeedForward, GroupMeta, LogitsOutput, Mixer, Norm, Part, PositionEncoding, StepContext,  # noqa: F401
                   TokenInput, Workspace)
from .registry import make_part, register_part  # noqa: F401
