"""Data: iterator protocol, synthetic generators, TFRecord input pipeline."""
from recml_b200.data.iterator import ArraySpec, IterableIterator, Iterator, TFDatasetIterator
from recml_b200.data.preprocessing import PreprocessingMode
from recml_b200.data.prefetch import DevicePrefetcher
