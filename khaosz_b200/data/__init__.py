from .dataset import BaseDataset, DatasetFactory, DPODataset, GRPODataset, SEQDataset, SFTDataset
from .sampler import ResumableDistributedSampler
from .storage import (H5Store, MmapStore, Store, StoreFactory, detect_format, load_bin, load_h5, save_bin,
                      save_h5)

__all__ = ["BaseDataset", "DatasetFactory", "DPODataset", "GRPODataset", "SEQDataset", "SFTDataset",
           "ResumableDistributedSampler", "H5Store", "MmapStore", "Store", "StoreFactory", "detect_format",
           "load_bin", "load_h5", "save_bin", "save_h5"]
