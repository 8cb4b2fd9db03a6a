from .parquet_dataset import DataConfig, StatefulParquetDataset
from .synthetic import SyntheticConfig, SyntheticTokenDataset

__all__ = ["DataConfig", "StatefulParquetDataset", "SyntheticConfig", "SyntheticTokenDataset"]
