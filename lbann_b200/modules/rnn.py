"""Recurrent cells (python/lbann/modules/rnn.py:8-456).

``LSTMCell`` is composed from a fully-connected layer and element-wise gates;
``GRU`` wraps the stacked-GRU layer (one kernel sequence per time step inside the layer);
``ChannelwiseGRU`` applies one GRU step independently to every channel.
"""
from __future__ import annotations

from ..frontend import core as L
from .base import ChannelwiseFullyConnectedModule, FullyConnectedModule, Module


class LSTMCell(Module):
    """One LSTM step: ``forward(x, (h, c)) -> (h', (h', c'))``."""

    global_count = 0

    def __init__(self, size, bias=True, weights=None, name=None, data_layout="data_parallel"):
        super().__init__()
        LSTMCell.global_count += 1
        self.step, self.size = 0, size
        self.name = name or f"lstmcell{LSTMCell.global_count}"
        self.data_layout = data_layout
        self.fc = FullyConnectedModule(4 * size, bias=bias, weights=weights, name=self.name + "_fc",
                                       data_layout=data_layout)

    def forward(self, x, prev_state):
        self.step += 1
        n = f"{self.name}_step{self.step}"
        h_prev, c_prev = prev_state
        z = self.fc(L.Concatenation([x, h_prev], name=n + "_input"))
        s = L.Slice(z, slice_points=[0, self.size, 2 * self.size, 3 * self.size, 4 * self.size],
                    name=n + "_slice")
        f = L.Sigmoid(L.Identity(s), name=n + "_forget_gate")
        i = L.Sigmoid(L.Identity(s), name=n + "_input_gate")
        o = L.Sigmoid(L.Identity(s), name=n + "_output_gate")
        g = L.Tanh(L.Identity(s), name=n + "_cell_update")
        c = L.Add(L.Multiply(f, c_prev), L.Multiply(i, g), name=n + "_cell")
        h = L.Multiply(o, L.Tanh(c), name=n + "_output")
        return h, (h, c)


class GRU(Module):
    """Stacked GRU over a whole ``[sequence, features]`` sample."""

    global_count = 0

    def __init__(self, size, bias=True, weights=None, name=None, num_layers=1):
        super().__init__()
        GRU.global_count += 1
        self.size, self.num_layers, self.instance = size, num_layers, 0
        self.name = name or f"gru{GRU.global_count}"
        ws = list(weights) if weights else []
        names = ("ih_matrix", "hh_matrix", "ih_bias", "hh_bias")
        while len(ws) < 4 * num_layers:
            li, k = divmod(len(ws), 4)
            init = L.UniformInitializer(min=-1 / size ** 0.5, max=1 / size ** 0.5)
            ws.append(L.Weights(initializer=init, name=f"{self.name}_layer{li}_{names[k]}"))
        self.weights = ws

    def forward(self, x, h0):
        self.instance += 1
        return L.GRU(x, h0, hidden_size=self.size, num_layers=self.num_layers, weights=self.weights,
                     name=f"{self.name}_instance{self.instance}")


class ChannelwiseGRU(Module):
    """One GRU step applied to every channel of ``[channels, size]`` tensors."""

    global_count = 0

    def __init__(self, num_channels, size, bias=True, weights=None, name=None):
        super().__init__()
        ChannelwiseGRU.global_count += 1
        self.step, self.size, self.channels = 0, size, num_channels
        self.name = name or f"channelwisegru{ChannelwiseGRU.global_count}"
        ws = list(weights) if weights else []
        self.ih = ChannelwiseFullyConnectedModule(3 * size, bias=bias, weights=ws[0:2] or None,
                                                  name=self.name + "_ih_fc")
        self.hh = ChannelwiseFullyConnectedModule(3 * size, bias=bias, weights=ws[2:4] or None,
                                                  name=self.name + "_hh_fc")

    def forward(self, x, h_prev):
        self.step += 1
        n = f"{self.name}_step{self.step}"
        S = self.size
        si = L.Slice(self.ih(x), axis=1, slice_points=[0, S, 2 * S, 3 * S], name=n + "_ih_slice")
        sh = L.Slice(self.hh(h_prev), axis=1, slice_points=[0, S, 2 * S, 3 * S], name=n + "_hh_slice")
        ir, iz, i_n = L.Identity(si), L.Identity(si), L.Identity(si)
        hr, hz, hn = L.Identity(sh), L.Identity(sh), L.Identity(sh)
        r = L.Sigmoid(L.Add(ir, hr), name=n + "_reset")
        z = L.Sigmoid(L.Add(iz, hz), name=n + "_update")
        cand = L.Tanh(L.Add(i_n, L.Multiply(r, hn)), name=n + "_candidate")
        one_minus_z = L.AddConstant(L.Scale(z, constant=-1.0), constant=1.0)
        return L.Add(L.Multiply(one_minus_z, cand), L.Multiply(z, h_prev), name=n + "_output")
