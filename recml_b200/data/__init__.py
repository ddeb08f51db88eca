"""Data: iterator protocol, synthetic generators, TFRecord input pipeline."""
from recml_b200.data.iterator import ArraySpec, IterableIterator, Iterator, TFDatasetIterator
from recml_b200.data.preprocessing import PreprocessingMode
from recml_b200.data.prefetch import DevicePrefetcher
from recml_b200.data.tfrecord_factory import (DatasetShardingInfo, FileFormat, FixedLenFeature, TFDatasetFactory,
                                              VarLenFeature)
