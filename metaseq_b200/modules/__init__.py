from .adaptive_softmax import AdaptiveSoftmax  # noqa: F401,E402
from .group_norm_fp32 import GroupNormFp32  # noqa: F401,E402
from .quant_noise import quant_noise  # noqa: F401,E402
