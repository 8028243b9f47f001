"""Dense gated feed-forward: down(act(gate(x)) * up(x)) (qwen_triton/modules/mlp.py:10-22, where act is SiLU;
here it is a parameter: any of ``kernels.ACTIVATIONS``).

gate and up run as one product over the fused weight [gate; up].  In bfloat16 its rows alternate 16 of gate and
16 of up, so that the GEMM for many tokens can apply the SiLU gate in its epilogue (one warp then holds both halves
of 16 features) and write the activation directly; few tokens take the split-K product and the separate kernel,
which reads the same layout.
"""
from __future__ import annotations

import torch

from ..ops import kernels
from ..ops.kernels import GemmOut
from ..weights.tensors import TensorSpec
from .base import DeferredProduct, Runtime, register_feed_forward, to_device
from .linear import Linear


@register_feed_forward("gated_mlp")
class GatedMLP:
    graph_safe = True

    def __init__(self, params, prefix: str, runtime: Runtime) -> None:
        self.prefix = prefix
        self.runtime = runtime
        self.hidden = int(params["hidden_size"])
        self.inter = int(params["intermediate_size"])
        self.activation = params.get("activation", "silu")
        if self.activation not in kernels.ACTIVATIONS:
            raise ValueError(f"{prefix}: gate activation {self.activation!r} is not one of {sorted(kernels.ACTIVATIONS)}")
        self.names = {k: params.get(k, f"{k}_proj") for k in ("gate", "up", "down")}
        fused = runtime.dtype == torch.bfloat16 and self.inter % kernels.SWIGLU_GROUP == 0 and self.hidden % 8 == 0
        self.group = kernels.SWIGLU_GROUP if fused else 0
        self.gate_up = Linear("mlp.gate_up", 2 * self.inter, self.hidden, runtime, role="gate")
        self.down = Linear("mlp.down", self.hidden, self.inter, runtime, role="mlp_out")
        runtime.workspace.declare("mlp.act", runtime.max_step_tokens * self.inter, runtime.dtype)
        # few tokens: the gate in the epilogue of the gate/up product, which then also applies the factor of the norm
        # in front of it (``ScaledRows``)
        self.takes_scaled_rows = bool(self.group) and self.gate_up.fused_capable

    @classmethod
    def expected_tensors(cls, params, prefix: str) -> dict[str, TensorSpec]:
        hidden, inter = int(params["hidden_size"]), int(params["intermediate_size"])
        n = {k: params.get(k, f"{k}_proj") for k in ("gate", "up", "down")}
        return {f"{prefix}.{n['gate']}.weight": TensorSpec((inter, hidden)),
                f"{prefix}.{n['up']}.weight": TensorSpec((inter, hidden)),
                f"{prefix}.{n['down']}.weight": TensorSpec((hidden, inter))}

    def load(self, source) -> None:
        n, p = self.names, self.prefix
        gate, up = source(f"{p}.{n['gate']}.weight"), source(f"{p}.{n['up']}.weight")
        self.gate_up.set_weight(kernels.interleave_gate_up(gate.to(self.runtime.dtype), up.to(self.runtime.dtype), self.group))
        self.down.set_weight(source(f"{p}.{n['down']}.weight"))

    def forward(self, x, ctx):
        tokens = x.shape[0]
        act = self.runtime.workspace.view("mlp.act", tokens, self.inter)
        if self.takes_scaled_rows and self.gate_up.fusable(tokens):
            self.gate_up.into_swiglu(x, act, self.activation)
        elif self.group and kernels.gemm_uses_pairs(x, self.gate_up.weight):
            kernels.gemm_tc_pair(x, self.gate_up.weight, GemmOut(act.view(1, tokens, self.inter)), swiglu=True, activation=self.activation)
        elif self.group and kernels.gemm_tc_supported(x, self.gate_up.weight) and self.gate_up.plan_splits(tokens) == 1:
            # a weight whose tiles fill the machine unsplit: the gate in the plain product's epilogue
            kernels.gemm_tc(x, self.gate_up.weight, GemmOut(act.view(1, tokens, self.inter)), swiglu=True, activation=self.activation)
        else:
            kernels.swiglu(self.gate_up(x), act, self.group, self.activation)
        # few tokens: the down projection is left to the norm behind it, which launches it with the residual addition
        # (and its own preparation) in the product's epilogue
        return DeferredProduct(self.down, act) if self.down.fusable(tokens) else self.down(act)


# Most (token, expert) pairs that run as matrix-vector passes, each streaming its expert's rows once: up to two pairs
# per expert, and never more than 64.  Beyond, pairs that share an expert would each read its weights again (from L2 at
# best), so the pairs are ordered by expert and the products run in tiles on the tensor cores, every expert read once
# (8 experts of 1,024 x 4,096 at 64 pairs: 0.77 ms a four-layer step per pair, against the dense model's 0.32).
_PAIRS_BY_PAIR = 64


@register_feed_forward("table_experts")
class TableExperts:
    """A set of small two-matrix feed-forward layers ("experts"), down_e(act(up_e(x))) without biases, of which every
    token runs the ``top`` that an integer table [vocab, top] names for its token id; their outputs are summed with
    the weight ``pair_weight`` each (default 1 / top, the mean).  There is no learned router: the choice depends on
    the token id alone, so it is read on the device from the step's token ids and a step launches the same kernels
    whatever the tokens are.

    Parameters: ``hidden_size``, ``expert_size`` (width of an expert's middle), ``experts``, ``top``, ``vocab_size``,
    ``activation`` (one of ``kernels.ACTIVATIONS``), and the tensor-name pieces ``table``, ``expert`` (a format of the
    expert's number), ``up``, ``down``, ``weight_suffix``.
    """

    graph_safe = True

    def __init__(self, params, prefix: str, runtime: Runtime) -> None:
        self.prefix = prefix
        self.runtime = runtime
        self.hidden = int(params["hidden_size"])
        self.inter = int(params["expert_size"])
        self.experts = int(params["experts"])
        self.top = int(params["top"])
        self.vocab = int(params["vocab_size"])
        self.activation = params.get("activation", "gelu")
        if self.activation not in kernels.ACTIVATIONS:
            raise ValueError(f"{prefix}: activation {self.activation!r} is not one of {sorted(kernels.ACTIVATIONS)}")
        if not 0 < self.top <= self.experts:
            raise ValueError(f"{prefix}: {self.top} experts per token out of {self.experts}")
        self.pair_weight = float(params.get("pair_weight", 1.0 / self.top))
        self.params = dict(params)
        self.up = self.down = self.table = None
        ws = runtime.workspace
        ws.declare("experts.out", runtime.max_step_tokens * self.hidden, torch.float32)
        # many tokens in bfloat16: the pairs ordered by expert in tiles of rows, both products on the tensor cores
        self.tiled = runtime.dtype == torch.bfloat16 and self.hidden % 8 == 0 and self.inter % 8 == 0
        pairs = runtime.max_step_tokens * self.top
        rows = pairs
        if self.tiled:
            tiles = kernels.expert_tiles(pairs, self.experts)
            rows = tiles * kernels.EXPERT_TILE_ROWS
            ws.declare("experts.ordered", rows * self.hidden, runtime.dtype)
            ws.declare("experts.y", rows * self.hidden, runtime.dtype)
            ws.declare("experts.route", pairs + rows + tiles, torch.int32)
        ws.declare("experts.mid", rows * self.inter, runtime.dtype)

    @staticmethod
    def _tensor_names(params, prefix: str) -> tuple[str, list[tuple[str, str]]]:
        suffix = str(params.get("weight_suffix", ".weight"))
        expert = str(params.get("expert", "experts.{}"))
        up, down = params.get("up", "up"), params.get("down", "down")
        pairs = [(f"{prefix}.{expert.format(e)}.{up}{suffix}", f"{prefix}.{expert.format(e)}.{down}{suffix}")
                 for e in range(int(params["experts"]))]
        return f"{prefix}.{params.get('table', 'table')}", pairs

    @classmethod
    def expected_tensors(cls, params, prefix: str) -> dict[str, TensorSpec]:
        hidden, inter = int(params["hidden_size"]), int(params["expert_size"])
        table, pairs = cls._tensor_names(params, prefix)
        out = {table: TensorSpec((int(params["vocab_size"]), int(params["top"])), role="table", table_high=int(params["experts"]))}
        for up, down in pairs:
            out[up] = TensorSpec((inter, hidden), init_std=0.05)
            out[down] = TensorSpec((hidden, inter), init_std=0.05)
        return out

    def load(self, source) -> None:
        table, pairs = self._tensor_names(self.params, self.prefix)
        dtype, device = self.runtime.dtype, self.runtime.device
        self.up = torch.stack([source(up).to(device=device, dtype=dtype) for up, _ in pairs]).contiguous()
        self.down = torch.stack([source(down).to(device=device, dtype=dtype) for _, down in pairs]).contiguous()
        table = source(table)
        if int(table.min()) < 0 or int(table.max()) >= self.experts:
            raise ValueError(f"{self.prefix}: the table names experts outside 0..{self.experts - 1}")
        self.table = to_device(table, torch.int32, device)

    def forward(self, x, ctx) -> GemmOut:
        tokens = x.shape[0]
        ws = self.runtime.workspace
        out = ws.view("experts.out", tokens, self.hidden)
        pairs = tokens * self.top
        if self.tiled and pairs > min(_PAIRS_BY_PAIR, 2 * self.experts):
            tiles = kernels.expert_tiles(pairs, self.experts)
            rows = tiles * kernels.EXPERT_TILE_ROWS
            kernels.experts_tiled(x, ctx.token_ids, self.table, self.up, self.down, ws.view("experts.ordered", rows, self.hidden),
                                  ws.view("experts.mid", rows, self.inter), ws.view("experts.y", rows, self.hidden),
                                  ws.view("experts.route", pairs + rows + tiles), out, self.activation, self.pair_weight)
        else:
            mid = ws.view("experts.mid", pairs, self.inter)
            kernels.experts_by_pair(x, ctx.token_ids, self.table, self.up, self.down, mid, out, self.activation, self.pair_weight)
        return GemmOut(out.view(1, tokens, self.hidden))
