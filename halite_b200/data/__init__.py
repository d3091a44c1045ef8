from .dataloader import DataLoader, DataManager, SimpleDataLoader
from .dataset import (HFDataset, MapDataset, SyntheticTokenDataset, WeightedIterableDataset,
                      build_dataset_from_spec)
from .record import Record
