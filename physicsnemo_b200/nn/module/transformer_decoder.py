"""Decoder-only transformer stack (parity: ``physicsnemo/nn/module/transformer_decoder.py``): layers of
self-attention → a second self-attention block (named ``multihead_attn`` for checkpoint compatibility)
→ feed-forward, pre- or post-norm; ``TransformerDecoder`` always runs them causally."""
import copy
from typing import Callable, Optional, Union

import torch
from torch import Tensor
from torch.nn import Dropout, LayerNorm, Linear, Module, ModuleList, MultiheadAttention
from torch.nn import functional as F


def _get_clones(module, N):
    return ModuleList([copy.deepcopy(module) for _ in range(N)])


def _get_activation_fn(activation: str) -> Callable[[Tensor], Tensor]:
    if activation == "relu":
        return F.relu
    if activation == "gelu":
        return F.gelu
    raise RuntimeError(f"activation should be relu/gelu, not {activation}")


class TransformerDecoder(Module):
    __constants__ = ["norm"]

    def __init__(self, decoder_layer, num_layers, norm=None):
        super().__init__()
        self.layers = _get_clones(decoder_layer, num_layers)
        self.num_layers, self.norm = num_layers, norm

    def forward(self, tgt: Tensor, tgt_mask: Optional[Tensor] = None, tgt_key_padding_mask: Optional[Tensor] = None,
                tgt_is_causal: Optional[bool] = None) -> Tensor:
        out = tgt
        for layer in self.layers:
            out = layer(out, tgt_mask=tgt_mask, tgt_key_padding_mask=tgt_key_padding_mask, tgt_is_causal=True)
        return self.norm(out) if self.norm is not None else out


class DecoderOnlyLayer(Module):
    __constants__ = ["norm_first"]

    def __init__(self, d_model: int, nhead: int, dim_feedforward: int = 2048, dropout: float = 0.1,
                 activation: Union[str, Callable[[Tensor], Tensor]] = F.relu, layer_norm_eps: float = 1e-5,
                 batch_first: bool = False, norm_first: bool = False, bias: bool = True, device=None, dtype=None) -> None:
        kw = {"device": device, "dtype": dtype}
        super().__init__()
        self.self_attn = MultiheadAttention(d_model, nhead, dropout=dropout, batch_first=batch_first, bias=bias, **kw)
        self.multihead_attn = MultiheadAttention(d_model, nhead, dropout=dropout, batch_first=batch_first, bias=bias, **kw)
        self.linear1 = Linear(d_model, dim_feedforward, bias=bias, **kw)
        self.dropout = Dropout(dropout)
        self.linear2 = Linear(dim_feedforward, d_model, bias=bias, **kw)
        self.norm_first = norm_first
        self.norm1 = LayerNorm(d_model, eps=layer_norm_eps, bias=bias, **kw)
        self.norm2 = LayerNorm(d_model, eps=layer_norm_eps, bias=bias, **kw)
        self.norm3 = LayerNorm(d_model, eps=layer_norm_eps, bias=bias, **kw)
        self.dropout1, self.dropout2, self.dropout3 = Dropout(dropout), Dropout(dropout), Dropout(dropout)
        self.activation = _get_activation_fn(activation) if isinstance(activation, str) else activation

    def __setstate__(self, state):
        state.setdefault("activation", F.relu)
        super().__setstate__(state)

    def _attend(self, attn, drop, x, mask, pad, causal):
        return drop(attn(x, x, x, attn_mask=mask, key_padding_mask=pad, is_causal=causal, need_weights=False)[0])

    def _sa_block(self, x, attn_mask, key_padding_mask, is_causal=False):
        return self._attend(self.self_attn, self.dropout1, x, attn_mask, key_padding_mask, is_causal)

    def _mha_block(self, x, attn_mask, key_padding_mask, is_causal=False):
        return self._attend(self.multihead_attn, self.dropout2, x, attn_mask, key_padding_mask, is_causal)

    def _ff_block(self, x):
        return self.dropout3(self.linear2(self.dropout(self.activation(self.linear1(x)))))

    def forward(self, tgt: Tensor, tgt_mask: Optional[Tensor] = None, tgt_key_padding_mask: Optional[Tensor] = None,
                tgt_is_causal: bool = False) -> Tensor:
        x = tgt
        a = (tgt_mask, tgt_key_padding_mask, tgt_is_causal)
        if self.norm_first:
            x = x + self._sa_block(self.norm1(x), *a)
            x = x + self._mha_block(self.norm2(x), *a)
            return x + self._ff_block(self.norm3(x))
        x = self.norm1(x + self._sa_block(x, *a))
        x = self.norm2(x + self._mha_block(x, *a))
        return self.norm3(x + self._ff_block(x))
