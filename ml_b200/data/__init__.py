from .loader import TokenLoader, BatchPipe, RawTokenLoader, write_token_bin, open_token_file, is_llmc_bin, read_raw_tokens  # noqa: F401
from .synthetic import bench_batch, mm_batch, random_pixels  # noqa: F401
