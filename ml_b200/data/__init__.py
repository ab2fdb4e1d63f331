from .loader import TokenLoader, BatchPipe, RawTokenLoader, write_token_bin  # noqa: F401
from .synthetic import bench_batch, mm_batch, random_pixels  # noqa: F401
