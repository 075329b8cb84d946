"""came_b200: the CAME optimizer step on NVIDIA B200 (sm_100a), a drop-in for the torch.optim classes of
tukisuwa/CAME (came_pytorch/__init__.py:1-8).  Importing the package loads libcame_b200.so; there is no
fallback path when it is missing."""
from . import _lib

_lib.load()

from .optim import CAME, CAMECUDA, CAME8bit, CAME8bit2D, CAME8bitFull, CAME8bitMemory  # noqa: E402

__all__ = ["CAME", "CAMECUDA", "CAME8bit", "CAME8bitMemory", "CAME8bitFull", "CAME8bit2D"]
