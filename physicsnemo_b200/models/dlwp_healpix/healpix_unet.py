"""DLWP U-Nets on the HEALPix mesh: feed-forward (``HEALPixUNet``) and recurrent (``HEALPixRecUNet``).

Parity: ``physicsnemo/models/dlwp_healpix/HEALPixUNet.py`` and ``HEALPixRecUNet.py`` — inputs are
``[prognostics (B, F, T, C, H, W), decoder inputs (B, F, T_total, C_d, H, W), constants (F, C_c, H, W), couplings]``;
every integration step folds time into channels and faces into the batch, runs encoder → decoder, unfolds to
``(B, F, T_in, C_out, H, W)``, optionally adds the input (residual prediction), applies output constraints and feeds the
prognostic channels back in; the recurrent variant re-initialises its hidden states every ``reset_cycle`` by replaying
``presteps`` earlier steps.  ``encoder`` / ``decoder`` are config mappings (``_target_`` …), classes or partials, see
``layers.build``.
"""
from __future__ import annotations

import re
from dataclasses import dataclass
from typing import Sequence

import torch

from ...core.meta import ModelMetaData
from ...core.module import Module
from ...nn.module.hpx import HEALPixFoldFaces, HEALPixUnfoldFaces
from .layers import _is_config, build


@dataclass
class MetaData(ModelMetaData):
    name: str = "DLWP_HEALPixUNet"
    jit: bool = False
    cuda_graphs: bool = True
    amp_cpu: bool = True
    amp_gpu: bool = True


def _hours(spec) -> int:
    """Hours of a duration like ``"6h"``, ``"1d"``, ``"90min"`` (pandas-style suffixes) or a number of hours."""
    if isinstance(spec, (int, float)):
        return int(spec)
    m = re.fullmatch(r"\s*(\d+(?:\.\d+)?)\s*([a-zA-Z]+)\s*", str(spec))
    if not m:
        raise ValueError(f"cannot parse duration {spec!r}")
    unit = m.group(2).lower()
    per_hour = {"h": 1.0, "hr": 1.0, "hour": 1.0, "hours": 1.0, "d": 24.0, "day": 24.0, "days": 24.0, "min": 1 / 60, "t": 1 / 60,
                "m": 1 / 60, "s": 1 / 3600, "w": 168.0}
    if unit not in per_hour:
        raise ValueError(f"unknown duration unit in {spec!r}")
    return int(float(m.group(1)) * per_hour[unit])


class _HEALPixBase(Module):
    _recurrent = False

    def __init__(self, encoder, decoder, input_channels, output_channels, n_constants, decoder_input_channels, input_time_dim,
                 output_time_dim, presteps=0, enable_nhwc=False, enable_healpixpad=False, couplings=(), residual_prediction=True,
                 couplings_time_first=True, constraints=None, is_diagnostic=False):
        super().__init__(meta=MetaData(name=type(self).__name__))
        self.channel_dim = 2
        couplings = list(couplings or [])
        if self._recurrent and n_constants == 0 and decoder_input_channels == 0:
            raise NotImplementedError("support for models with no constant fields and no decoder inputs (TOA insolation) is not available at this time.")
        if couplings:
            if n_constants == 0:
                raise NotImplementedError("support for coupled models with no constant fields is not available at this time.")
            if decoder_input_channels == 0:
                raise NotImplementedError("support for coupled models with no decoder inputs (TOA insolation) is not available at this time.")
        self.coupled_channels = sum(len(c["params"]["variables"]) * len(c["params"]["input_times"]) for c in couplings)
        self.couplings, self.train_couplers = couplings, None
        self.input_channels, self.output_channels = input_channels, output_channels
        self.n_constants, self.decoder_input_channels = n_constants, decoder_input_channels
        self.input_time_dim, self.output_time_dim = input_time_dim, output_time_dim
        self.presteps = presteps
        self.enable_nhwc, self.enable_healpixpad = enable_nhwc, enable_healpixpad
        self.residual_prediction, self.couplings_time_first, self.is_diagnostic = residual_prediction, couplings_time_first, is_diagnostic
        if is_diagnostic and output_time_dim != 1:
            raise ValueError(f"A diagnostic model (is_diagnostic=True) must have output_time_dim == 1 (got {output_time_dim}).")
        if residual_prediction and is_diagnostic:
            raise ValueError("A diagnostic model cannot predict a residual. Please set residual_prediction to False when is_diagnostic is True.")
        if not is_diagnostic and output_time_dim % input_time_dim != 0:
            raise ValueError(f"'output_time_dim' must be a multiple of 'input_time_dim' (got {output_time_dim} and {input_time_dim})")
        self.fold, self.unfold = HEALPixFoldFaces(), HEALPixUnfoldFaces(num_faces=12)
        self.encoder = build(encoder, input_channels=self._compute_input_channels(), enable_nhwc=enable_nhwc, enable_healpixpad=enable_healpixpad)
        self.encoder_depth = len(self.encoder.n_channels)
        self.decoder = build(decoder, output_channels=self._compute_output_channels(), enable_nhwc=enable_nhwc, enable_healpixpad=enable_healpixpad)
        self.constraints = None
        self.set_constraints(constraints)

    @property
    def integration_steps(self) -> int:
        return max(self.output_time_dim // self.input_time_dim, 1)

    def _compute_input_channels(self) -> int:
        return self.input_time_dim * (self.input_channels + self.decoder_input_channels) + self.n_constants + self.coupled_channels

    def _compute_output_channels(self) -> int:
        return (1 if self.is_diagnostic else self.input_time_dim) * self.output_channels

    def set_constraints(self, constraints=None):
        if constraints is not None:
            items = [constraints[k] for k in constraints.keys()] if _is_config(constraints) else list(constraints)
            self.constraints = torch.nn.ModuleList([build(c) for c in items])

    def _reshape_inputs(self, inputs: Sequence, step: int = 0) -> torch.Tensor:
        cd, T = self.channel_dim, self.input_time_dim
        flat = lambda t: t.flatten(start_dim=cd, end_dim=cd + 1)  # noqa: E731
        window = lambda t: flat(t[:, :, step * T:(step + 1) * T])  # noqa: E731
        batched = lambda t: t.expand(inputs[0].shape[0], *([-1] * t.dim()))  # noqa: E731
        if self.couplings:
            parts = [flat(inputs[0]), window(inputs[1]), batched(inputs[2]),
                     inputs[3].permute(0, 2, 1, 3, 4) if self.couplings_time_first else inputs[3]]
        elif self.n_constants == 0 and self.decoder_input_channels == 0:
            return self.fold(flat(inputs[0]))
        elif self.n_constants == 0:
            return self.fold(torch.cat([flat(inputs[0]), window(inputs[1])], dim=cd))
        elif self.decoder_input_channels == 0:
            return self.fold(torch.cat([flat(inputs[0]), batched(inputs[1])], dim=cd))
        else:
            parts = [flat(inputs[0]), window(inputs[1]), batched(inputs[2])]
        res = self.fold(torch.cat(parts, dim=cd))
        if self.enable_nhwc and self._recurrent:
            res = res.to(memory_format=torch.channels_last)
        return res

    def _reshape_outputs(self, outputs: torch.Tensor) -> torch.Tensor:
        outputs = self.unfold(outputs)
        s = tuple(outputs.shape)
        return outputs.reshape(s[0], s[1], 1 if self.is_diagnostic else self.input_time_dim, -1, *s[3:])

    def _step_input(self, inputs, outputs, step: int, offset: int):
        """Network input of integration step ``step`` (``offset`` = number of leading time windows to skip)."""
        if step == 0:
            s, T = offset, self.input_time_dim
            first = inputs[0][:, :, s * T:(s + 1) * T]
        else:
            s, first = step + offset, outputs[-1][:, :, :, :self.input_channels]
        rest = list(inputs[1:3]) + [inputs[3][s]] if self.couplings else list(inputs[1:])
        return self._reshape_inputs([first] + rest, step=s)

    def _advance(self, input_tensor, conditions_cln):
        kw = {"conditions_cln": conditions_cln} if conditions_cln is not None else {}
        combined = self._reshape_outputs(self.decoder(self.encoder(input_tensor, **kw), **kw))
        prognostics = combined[:, :, :, :self.input_channels]
        if self.residual_prediction:
            prognostics = prognostics + self._reshape_outputs(input_tensor[:, :self.input_channels * self.input_time_dim])
        out = torch.cat([prognostics, combined[:, :, :, self.input_channels:]], dim=3)
        if self.constraints is not None:
            for constraint in self.constraints:
                out = constraint(out)
        return out

    def _check(self, inputs):
        if not torch.compiler.is_compiling() and inputs[0].ndim != 6:
            raise ValueError(f"{type(self).__name__}.forward expects prognostics shaped (B, F, T, C, H, W)")


class HEALPixUNet(_HEALPixBase):
    """Feed-forward DLWP U-Net on the HEALPix mesh."""

    def forward(self, inputs: Sequence, output_only_last: bool = False, conditions_cln=None) -> torch.Tensor:
        self._check(inputs)
        outputs = []
        for step in range(self.integration_steps):
            x = self._step_input(inputs, outputs, step, 0)
            outputs.append(self._advance(x, conditions_cln[step] if conditions_cln is not None else None))
        return outputs[-1] if output_only_last else torch.cat(outputs, dim=self.channel_dim)


class HEALPixRecUNet(_HEALPixBase):
    """Recurrent DLWP U-Net on the HEALPix mesh (ConvGRU blocks in the decoder keep state between steps)."""

    _recurrent = True

    def __init__(self, encoder, decoder, input_channels, output_channels, n_constants, decoder_input_channels, input_time_dim,
                 output_time_dim, delta_time="6h", reset_cycle="24h", presteps=1, enable_nhwc=False, enable_healpixpad=False,
                 couplings=(), residual_prediction=True, couplings_time_first=True, constraints=None, is_diagnostic=False):
        super().__init__(encoder, decoder, input_channels, output_channels, n_constants, decoder_input_channels, input_time_dim,
                         output_time_dim, presteps, enable_nhwc, enable_healpixpad, couplings, residual_prediction,
                         couplings_time_first, constraints, is_diagnostic)
        self.delta_t, self.reset_cycle = _hours(delta_time), _hours(reset_cycle)

    def reset(self):
        self.encoder.reset()
        self.decoder.reset()

    def _initialize_hidden(self, inputs, outputs, step: int, conditions_cln=None) -> None:
        self.reset()
        T = self.input_time_dim
        for prestep in range(self.presteps):
            if step < self.presteps:
                s = step + prestep
                first = inputs[0][:, :, s * T:(s + 1) * T]
                rest = list(inputs[1:3]) + [inputs[3][prestep]] if self.couplings else list(inputs[1:])
                x = self._reshape_inputs([first] + rest, step=step + prestep)
            else:
                s = step - self.presteps + prestep
                first = outputs[s - 1][:, :, :, :self.input_channels]
                rest = list(inputs[1:3]) + [inputs[3][step - (prestep - self.presteps)]] if self.couplings else list(inputs[1:])
                x = self._reshape_inputs([first] + rest, step=s + 1)
            kw = {"conditions_cln": conditions_cln} if conditions_cln is not None else {}
            self.decoder(self.encoder(x, **kw), **kw)

    def forward(self, inputs: Sequence, output_only_last: bool = False, conditions_cln=None) -> torch.Tensor:
        self._check(inputs)
        self.reset()
        outputs = []
        for step in range(self.integration_steps):
            cond = conditions_cln[step] if conditions_cln is not None else None
            if (step * (self.delta_t * self.input_time_dim)) % self.reset_cycle == 0:
                self._initialize_hidden(inputs, outputs, step, cond)
            x = self._step_input(inputs, outputs, step, self.presteps)
            outputs.append(self._advance(x, cond))
        return outputs[-1] if output_only_last else torch.cat(outputs, dim=self.channel_dim)
