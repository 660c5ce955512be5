"""Model building: modules, layers, transformer blocks, recurrent and graph layers, losses."""
from .module import *  # noqa: F401,F403
from .module import Module, Sequential, Linear, manual_seed  # noqa: F401
from .transformer import (RotaryEmbedding, KVCache, SelfAttention, MultiheadAttention, MLP, GatedMLP,  # noqa: F401
                          DecoderBlock, TransformerEncoderLayer)
from .rnn import RNN, LSTM, GRU  # noqa: F401
from .gnn import Graph, GCNConv, SAGEConv, GATConv  # noqa: F401
from . import loss  # noqa: F401
