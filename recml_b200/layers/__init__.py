"""Model layers (the reference keeps them under `recml/layers/keras` and `recml/layers/linen`)."""
from recml_b200.layers.bert4rec import BERT4Rec, MaskedLMHead
from recml_b200.layers.dcn import CrossNetwork
from recml_b200.layers.dense import MLP, Linear
from recml_b200.layers.embeddings import PositionEmbedding, ReversibleEmbedding
from recml_b200.layers.hstu import (HSTU, HSTUBlock, RelativeBucketedTimeAndPositionBasedBias,
                                    RelativePositionalBias)
from recml_b200.layers.mamba import Mamba2, Mamba2Block, Mamba2Stack, Mamba4Rec
from recml_b200.layers.parallel import ColumnParallelLinear, RowParallelLinear, TensorParallelMLP
from recml_b200.layers.sasrec import SASRec
from recml_b200.layers.transformer import MultiHeadAttention, TransformerBlock
