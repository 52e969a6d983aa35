"""Drop-in name: ``import nvfp4_gemm`` gives the B200-native implementation."""
from nvfp4_cutlass_b200 import *  # noqa: F401,F403
from nvfp4_cutlass_b200 import _C, layout, __version__, __all__  # noqa: F401
