import torch  # noqa: F401  (loads libtorch before the extension)
from . import kernel  # noqa: F401
