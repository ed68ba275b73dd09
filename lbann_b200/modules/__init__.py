"""``lbann.modules``: reusable layer patterns with shared weights."""
from .base import (ChannelwiseFullyConnectedModule, Convolution2dModule, Convolution3dModule,  # noqa: F401
                   ConvolutionModule, FullyConnectedModule, Module)
from .activations import Gelu, Gelu_approx, Silu  # noqa: F401
from .graph import (DenseGCNConv, DenseGINConv, DenseGraphConv, DenseNNConv, GatedGraphConv, GCNConv,  # noqa: F401
                    GINConv, GraphConv, GraphExpand, GraphReduce, NNConv, SparseGINConv)
from .rnn import GRU, ChannelwiseGRU, LSTMCell  # noqa: F401
from .transformations import Cumsum, PeriodicPadding2D, PeriodicPadding3D, Permute  # noqa: F401
from . import transformer  # noqa: F401
from .transformer import (LearnedInputEncoding, MultiheadAttention, PositionalEncoding,  # noqa: F401
                          RotaryPositionalEmbedding, SequenceEncoding)
