"""B200-native displaced-patch-parallel SDXL UNet hot path (drop-in for the
corresponding part of sekstini/basedxl).  Importing the package needs no GPU;
running any operator needs an sm_100a device and the in-tree CUDA library."""
from .model import BasedXLPipeline  # noqa: F401
from .utils import BasedXLConfig, PatchParallelismCommManager  # noqa: F401
