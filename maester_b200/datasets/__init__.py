from maester_b200.datasets.experimental_otf import (  # noqa: F401
    Buffer_Dataset,
    Checkpoint_Dataset,
    Preload_Buffer_Dataset,
    Preprocess_Dataset,
    causal_lm,
)
from maester_b200.datasets.parquet_dataset import ParquetDataset, Sampling_Dataset, Scalable_Shard_Dataset  # noqa: F401
from maester_b200.datasets.builder import build_experimental_data_loader, parse_data_args  # noqa: F401
from maester_b200.datasets.synthetic import SyntheticLoader, build_synthetic_data_loader  # noqa: F401
