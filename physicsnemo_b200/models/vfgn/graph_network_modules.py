"""VFGN (virtual-foundry graph network): a learned particle simulator for sintering deformation.

Parity: ``physicsnemo/models/vfgn/graph_network_modules.py`` (``MLPNet`` with its lazily created
first layer ``lin_s``, ``EncoderNet``, ``EdgeBlock``, ``NodeBlock``, ``InteractionNet``,
``ResInteractionNet``, ``DecoderNet``, ``EncodeProcessDecode`` with optional placement of the
message-passing steps on several devices, ``VFGNLearnedSimulator`` with feature encoding /
decoding, random-walk noise, training ``forward`` and roll-out ``inference``).  Aggregation onto
nodes uses ``index_reduce`` / ``index_add`` instead of ``torch_scatter``; per-graph global context
is expanded with one ``repeat_interleave``; edge lists of a batch are offset with array
operations instead of a Python loop over graphs.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Literal

import numpy as np
import torch
import torch.nn.functional as F
from torch import Tensor
from torch.nn import Embedding, Linear, ReLU
from torch.utils.checkpoint import checkpoint

from ...core import Module
from ...core.meta import ModelMetaData

STD_EPSILON = 1e-8


@dataclass
class MetaData(ModelMetaData):
    name: str = "VFGNLearnedSimulator"
    jit: bool = False
    cuda_graphs: bool = True
    amp_cpu: bool = False
    amp_gpu: bool = False
    onnx_cpu: bool = False
    onnx_gpu: bool = False
    onnx_runtime: bool = False
    var_dim: int = 1
    func_torch: bool = False
    auto_grad: bool = False


def _need_2d(**tensors) -> None:
    if torch.compiler.is_compiling():
        return
    for name, t in tensors.items():
        if t.ndim != 2:
            raise ValueError(f"Expected {name} to be a 2D tensor, got shape {tuple(t.shape)}")


def _need_1d(**tensors) -> None:
    if torch.compiler.is_compiling():
        return
    for name, t in tensors.items():
        if t.ndim != 1:
            raise ValueError(f"Expected {name} to be a 1D index tensor, got shape {tuple(t.shape)}")


def scatter_reduce(src: Tensor, index: Tensor, dim_size: int, reduce: str = "add") -> Tensor:
    """Reduce rows of ``src`` into ``dim_size`` rows by ``index`` (``add | sum | mean | min | max | mul``)."""
    out = src.new_zeros((dim_size, *src.shape[1:]))
    if reduce in ("add", "sum"):
        return out.index_add_(0, index, src)
    name = {"mean": "mean", "min": "amin", "max": "amax", "mul": "prod"}.get(reduce)
    if name is None:
        raise ValueError(f"unknown aggregation {reduce!r}")
    return out.index_reduce_(0, index, src, name, include_self=False)


class MLPNet(Module):
    """ReLU MLP whose first layer is created at the first call from the input width (``lin_s``)."""

    def __init__(self, mlp_hidden_size: int = 128, mlp_num_hidden_layers: int = 2, output_size: int = 128,
                 layer_norm: bool = True):
        if not (mlp_hidden_size >= 0 and mlp_num_hidden_layers >= 0 and output_size >= 0):
            raise ValueError("Invalid arch params")
        super().__init__(meta=MetaData(name="vfgn_mlpnet"))
        self.mlp_hidden_size = mlp_hidden_size
        self.lins = torch.nn.ModuleList([Linear(mlp_hidden_size, mlp_hidden_size)
                                         for _ in range(max(mlp_num_hidden_layers - 1, 0))])
        self.lin_e = Linear(mlp_hidden_size, output_size)
        self.layer_norm = layer_norm
        self.relu = ReLU()

    def dynamic(self, name: str, module_class, *args, **kwargs):
        if not hasattr(self, name):
            self.add_module(name, module_class(*args, **kwargs))
        return getattr(self, name)

    def forward(self, x):
        _need_2d(x=x)
        lin_s = self.dynamic("lin_s", Linear, x.shape[-1], self.mlp_hidden_size).to(x.device)
        x = self.relu(lin_s(x))
        for lin in self.lins:
            x = self.relu(lin(x))
        x = self.lin_e(x)
        return F.layer_norm(x, x.shape[1:]) if self.layer_norm else x


class EncoderNet(Module):
    def __init__(self, mlp_hidden_size: int = 128, mlp_num_hidden_layers: int = 2, latent_size: int = 128):
        if not (mlp_hidden_size >= 0 and mlp_num_hidden_layers >= 0 and latent_size >= 0):
            raise ValueError("Invalid arch params - EncoderNet")
        super().__init__(meta=MetaData(name="vfgn_encoder"))
        self._mlp_hidden_size, self._mlp_num_hidden_layers = mlp_hidden_size, mlp_num_hidden_layers
        self.edge_mlp = MLPNet(mlp_hidden_size, mlp_num_hidden_layers, latent_size)
        self.node_mlp = MLPNet(mlp_hidden_size, mlp_num_hidden_layers, latent_size)

    def forward(self, node_attr, edge_attr):
        _need_2d(node_attr=node_attr, edge_attr=edge_attr)
        return self.node_mlp(node_attr), self.edge_mlp(edge_attr)


class EdgeBlock(Module):
    def __init__(self, mlp_hidden_size, mlp_num_hidden_layers, latent_size, node_dim=0, use_receiver_nodes=True,
                 use_sender_nodes=True):
        super().__init__(meta=MetaData(name="vfgn_edgeblock"))
        self.node_dim = node_dim
        self._edge_model = MLPNet(mlp_hidden_size, mlp_num_hidden_layers, latent_size)
        self.use_receiver_nodes, self.use_sender_nodes = use_receiver_nodes, use_sender_nodes

    def forward(self, node_attr, edge_attr, receivers, senders):
        _need_2d(node_attr=node_attr, edge_attr=edge_attr)
        _need_1d(receivers=receivers, senders=senders)
        parts = [edge_attr]
        if self.use_receiver_nodes:
            parts.append(node_attr[receivers])
        if self.use_sender_nodes:
            parts.append(node_attr[senders])
        return node_attr, self._edge_model(torch.cat(parts, dim=-1)), receivers, senders


class NodeBlock(Module):
    def __init__(self, mlp_hidden_size, mlp_num_hidden_layers, latent_size,
                 aggr: Literal["add", "sum", "mean", "min", "max", "mul"] = "add", node_dim=0, use_received_edges=True,
                 use_sent_edges=False):
        super().__init__(meta=MetaData(name="vfgn_nodeblock"))
        self.aggr, self.node_dim = aggr, node_dim
        self.use_received_edges, self.use_sent_edges = use_received_edges, use_sent_edges
        self._node_model = MLPNet(mlp_hidden_size, mlp_num_hidden_layers, latent_size)

    def forward(self, x, edge_attr, receivers, senders):
        _need_2d(x=x, edge_attr=edge_attr)
        _need_1d(receivers=receivers, senders=senders)
        parts, n = [x], x.shape[0]
        # "aggr" may arrive as something else than a name through InteractionNet's positional call: default to a sum
        aggr = self.aggr if isinstance(self.aggr, str) else "add"
        if self.use_received_edges:
            parts.append(scatter_reduce(edge_attr, receivers, n, aggr))
        if self.use_sent_edges:
            parts.append(scatter_reduce(edge_attr, senders, n, aggr))
        return self._node_model(torch.cat(parts, dim=-1)), edge_attr, receivers, senders


class InteractionNet(torch.nn.Module):
    def __init__(self, mlp_hidden_size, mlp_num_hidden_layers, latent_size,
                 aggr: Literal["add", "sum", "mean", "min", "max", "mul"] = "add", node_dim=0):
        super().__init__()
        self._edge_block = EdgeBlock(mlp_hidden_size, mlp_num_hidden_layers, latent_size, node_dim)
        self._node_block = NodeBlock(mlp_hidden_size, mlp_num_hidden_layers, latent_size, aggr, node_dim)

    def forward(self, x, edge_attr, receivers, senders):
        _need_2d(x=x, edge_attr=edge_attr)
        _need_1d(receivers=receivers, senders=senders)
        if x.shape[-1] != edge_attr.shape[-1]:
            raise ValueError("node feature size should equal to edge feature size")
        return self._node_block(*self._edge_block(x, edge_attr, receivers, senders))


class ResInteractionNet(torch.nn.Module):
    def __init__(self, mlp_hidden_size, mlp_num_hidden_layers, latent_size,
                 aggr: Literal["add", "sum", "mean", "min", "max", "mul"] = "add", node_dim=0):
        super().__init__()
        self.itn = InteractionNet(mlp_hidden_size, mlp_num_hidden_layers, latent_size, aggr, node_dim)

    def forward(self, x, edge_attr, receivers, senders):
        dx, de, receivers, senders = self.itn(x, edge_attr, receivers, senders)
        return x + dx, edge_attr + de, receivers, senders


class DecoderNet(Module):
    def __init__(self, mlp_hidden_size, mlp_num_hidden_layers, output_size):
        if not (mlp_hidden_size >= 0 and mlp_num_hidden_layers >= 0 and output_size >= 0):
            raise ValueError("Invalid arch params - DecoderNet")
        super().__init__(meta=MetaData(name="vfgn_decoder"))
        self.mlp = MLPNet(mlp_hidden_size, mlp_num_hidden_layers, output_size, layer_norm=False)

    def forward(self, x):
        _need_2d(x=x)
        return self.mlp(x)


class EncodeProcessDecode(Module):
    def __init__(self, latent_size, mlp_hidden_size, mlp_num_hidden_layers, num_message_passing_steps, output_size,
                 device_list=None):
        if not (latent_size > 0 and mlp_hidden_size > 0 and mlp_num_hidden_layers > 0):
            raise ValueError("Invalid arch params - EncodeProcessDecode")
        if not num_message_passing_steps > 0:
            raise ValueError("Invalid arch params - EncodeProcessDecode")
        super().__init__(meta=MetaData(name="vfgn_encoderprocess_decode"))
        self.device_list = ["cpu"] if device_list is None else device_list
        self._encoder_network = EncoderNet(mlp_hidden_size, mlp_num_hidden_layers, latent_size)
        self._processor_networks = torch.nn.ModuleList(
            [InteractionNet(mlp_hidden_size, mlp_num_hidden_layers, latent_size) for _ in range(num_message_passing_steps)])
        self._decoder_network = DecoderNet(mlp_hidden_size, mlp_num_hidden_layers, output_size)

    def set_device(self, device_list):
        self.device_list = device_list

    def forward(self, x, edge_attr, receivers, senders):
        _need_2d(x=x, edge_attr=edge_attr)
        _need_1d(receivers=receivers, senders=senders)
        x, edge_attr = self._encoder_network(x, edge_attr)
        cur_x, cur_e = x, edge_attr
        origin = x.device
        spread = len(self.device_list) > 1 or str(self.device_list[0]) != str(origin.type)
        per_device = max(len(self._processor_networks) // max(len(self.device_list), 1), 1)
        for k, net in enumerate(self._processor_networks):
            if spread and self.device_list:
                dev = self.device_list[min(k // per_device, len(self.device_list) - 1)]
                if str(dev) != "cpu" or origin.type == "cpu":
                    net = net.to(dev)
                    cur_x, cur_e, receivers, senders = (t.to(dev) for t in (cur_x, cur_e, receivers, senders))
            if torch.is_grad_enabled() and cur_x.requires_grad:
                dx, de, receivers, senders = checkpoint(net, cur_x, cur_e, receivers, senders, use_reentrant=False)
            else:
                dx, de, receivers, senders = net(cur_x, cur_e, receivers, senders)
            # every step adds its update to the ENCODER output (not to the previous step's), as in the reference
            cur_x, cur_e = x.to(dx.device) + dx, edge_attr.to(de.device) + de
        return self._decoder_network(cur_x.to(origin))


class VFGNLearnedSimulator(Module):
    def __init__(self, num_dimensions: int = 3, num_seq: int = 5, boundaries=None, num_particle_types: int = 3,
                 particle_type_embedding_size: int = 16, normalization_stats=None,
                 graph_mode: Literal["radius", "knn"] = "radius", connectivity_param: float = 0.015):
        if not (num_dimensions >= 0 and num_seq >= 3):
            raise ValueError("Invalid arch params - VFGNLearnedSimulator")
        super().__init__(meta=MetaData(name="vfgn_simulator"))
        self._latent_size, self._mlp_hidden_size, self._mlp_num_hidden_layers = 128, 128, 2
        self._num_message_passing_steps = 10
        self._num_dimensions, self._num_seq = num_dimensions, num_seq
        self._connectivity_param = connectivity_param
        self._boundaries, self._normalization_stats = boundaries, normalization_stats
        self.graph_mode = graph_mode
        self._graph_network = EncodeProcessDecode(self._latent_size, self._mlp_hidden_size, self._mlp_num_hidden_layers,
                                                  self._num_message_passing_steps, self._num_dimensions)
        self._num_particle_types = num_particle_types
        self.embedding = Embedding(num_particle_types + 1, particle_type_embedding_size)
        self.message_passing_devices = []

    def setMessagePassingDevices(self, devices):
        self.message_passing_devices = devices

    def to(self, device):
        new_self = super().to(device)
        if isinstance(self._boundaries, torch.Tensor):
            new_self._boundaries = self._boundaries.to(device)
        for key, stats in (self._normalization_stats or {}).items():
            if hasattr(stats, "to"):
                moved = stats.to(device)
                if moved is not None:
                    new_self._normalization_stats[key] = moved
        if str(device) != "cpu" and self.message_passing_devices:
            self._graph_network.set_device(self.message_passing_devices)
        return new_self

    @staticmethod
    def time_diff(input_seq):
        return input_seq[:, 1:] - input_seq[:, :-1]

    def _compute_connectivity_for_batch(self, senders_list, receivers_list, n_node, n_edge):
        """Offset the per-graph edge indices of a batch by the node counts of the preceding graphs."""
        n_node, n_edge = np.asarray(n_node).reshape(-1), np.asarray(n_edge).reshape(-1)
        offsets = np.repeat(np.concatenate([[0], np.cumsum(n_node[:-1])]), n_edge)
        return ((np.asarray(senders_list) + offsets).astype(np.int32), (np.asarray(receivers_list) + offsets).astype(np.int32))

    def get_random_walk_noise_for_position_sequence(self, position_sequence, noise_std_last_step):
        vel = self.time_diff(position_sequence)
        noise = torch.empty(vel.shape, dtype=vel.dtype).normal_(mean=0, std=noise_std_last_step / vel.shape[1] ** 0.5)
        noise = torch.cumsum(noise, dim=1)
        return torch.cat([torch.zeros_like(noise[:, 0:1]), torch.cumsum(noise, dim=1)], dim=1)

    def EncodingFeature(self, position_sequence, n_node, n_edge, senders_list, receivers_list, global_context, particle_types):
        dev = position_sequence.device
        last = position_sequence[:, -1]
        vel = self.time_diff(position_sequence)
        acc = self.time_diff(vel)
        s, r = self._compute_connectivity_for_batch(senders_list.detach().cpu().numpy(), receivers_list.detach().cpu().numpy(),
                                                    n_node.detach().cpu().numpy(), n_edge.detach().cpu().numpy())
        senders, receivers = torch.as_tensor(s, dtype=torch.long, device=dev), torch.as_tensor(r, dtype=torch.long, device=dev)
        vs, as_ = self._normalization_stats["velocity"], self._normalization_stats["acceleration"]
        nodes = [((vel - vs.mean) / vs.std)[:, -1].reshape(vel.shape[0], -1), ((acc - as_.mean) / as_.std).reshape(acc.shape[0], -1)]
        if self._num_particle_types > 1:
            nodes.append(self.embedding(particle_types))
        disp = (last.index_select(0, senders) - last.index_select(0, receivers)) / self._connectivity_param
        edges = [disp, torch.norm(disp, dim=-1, keepdim=True)]
        if global_context is not None:
            cs = self._normalization_stats["context"]
            ctx = (global_context - cs.mean) / torch.maximum(cs.std, torch.tensor([STD_EPSILON], device=cs.std.device))
            ctx = torch.repeat_interleave(ctx, n_node.to(torch.long).reshape(-1).to(ctx.device), dim=0)
            nodes.append(ctx.reshape(ctx.shape[0], -1).to(dev))
        return torch.cat(nodes, -1).float(), torch.cat(edges, -1).float(), senders, receivers

    def DecodingFeature(self, normalized_accelerations, position_sequence, predict_length):
        st = self._normalization_stats["acceleration"]
        acc = normalized_accelerations.double().reshape(-1, predict_length, 3) * st.std + st.mean
        vel = (position_sequence[:, -1] - position_sequence[:, -2]).unsqueeze(1) + torch.cumsum(acc, dim=1)
        return position_sequence[:, -1].unsqueeze(1) + torch.cumsum(vel, dim=1)

    def _inverse_decoder_postprocessor(self, next_positions, position_sequence):
        previous = torch.cat([position_sequence[:, -2:], next_positions[:, :-1]], dim=1)
        positions = torch.cat([position_sequence[:, -1].unsqueeze(1), next_positions], dim=1)
        vel = positions - previous
        st = self._normalization_stats["acceleration"]
        return (((vel[:, 1:] - vel[:, :-1]) - st.mean) / st.std).reshape(-1, self._num_dimensions).float()

    def inference(self, position_sequence: Tensor, n_particles_per_example, n_edges_per_example, senders, receivers,
                  predict_length, global_context=None, particle_types=None) -> Tensor:
        graph = self.EncodingFeature(position_sequence, n_particles_per_example, n_edges_per_example, senders, receivers,
                                     global_context, particle_types)
        return self.DecodingFeature(self._graph_network(*graph), position_sequence, predict_length)

    def forward(self, next_positions: Tensor, position_sequence_noise: Tensor, position_sequence: Tensor,
                n_particles_per_example, n_edges_per_example, senders: Tensor, receivers: Tensor, predict_length,
                global_context=None, particle_types=None):
        if not torch.compiler.is_compiling():
            if position_sequence.ndim != 3 or position_sequence_noise.ndim != 3:
                raise ValueError("Expected position_sequence and position_sequence_noise to be 3D (N_nodes, T, D), got "
                                 f"{tuple(position_sequence.shape)} and {tuple(position_sequence_noise.shape)}")
            _need_1d(receivers=receivers, senders=senders)
        noisy = position_sequence + position_sequence_noise
        graph = self.EncodingFeature(noisy, n_particles_per_example, n_edges_per_example, senders, receivers,
                                     global_context, particle_types)
        predicted = self._graph_network(*graph)
        last_noise = position_sequence_noise[:, -1].unsqueeze(1).expand(-1, predict_length, -1)
        nxt = next_positions if next_positions.ndim == 3 else next_positions.unsqueeze(1)
        return predicted, self._inverse_decoder_postprocessor(nxt + last_noise, noisy)

    def get_normalized_acceleration(self, acceleration, predict_length):
        st = self._normalization_stats["acceleration"]
        return torch.tile((acceleration - st.mean) / st.std, [predict_length])
