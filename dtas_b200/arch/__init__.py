from .arch_base import Arch  # noqa: F401
from .b200 import B200  # noqa: F401
from .rtx3090 import RTX3090  # noqa: F401
