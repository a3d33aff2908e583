from maester_b200.parallel.parallel_dims import ParallelDims  # noqa: F401
from maester_b200.parallel.parallelize import (  # noqa: F401
    materialize,
    parallelize,
    parallelize_deepseek,
    parallelize_gemma,
    parallelize_llama,
)
