"""Model layers."""
from recml_b200.layers.dcn import CrossNetwork
from recml_b200.layers.dense import MLP, Linear
