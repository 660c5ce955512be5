"""Model building: modules, layers, transformer blocks, recurrent and graph layers, losses."""
from .module import *  # noqa: F401,F403
from .module import Module, Sequential, Linear, manual_seed  # noqa: F401
from .transformer import (RotaryEmbedding, KVCache, SelfAttention, MultiheadAttention, MLP, GatedMLP,  # noqa: F401
                          DecoderBlock, TransformerEncoderLayer)
from .rnn import RNN, LSTM, GRU  # noqa: F401
from .gnn import Graph, GCNConv, SAGEConv, GATConv  # noqa: F401
from . import loss  # noqa: F401

LoRA = LoRALinear          # the reference's name for the adapter layer


def LogSoftmax(dim=-1):
    from .module import _Fn
    from .. import tensor as _T
    return _Fn(lambda x: _T.log_softmax(x, dim))
