from .gemm import gemm  # noqa: F401
from .status import check_status, device_status  # noqa: F401
