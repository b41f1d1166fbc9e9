"""The training-step projection set of a GPT-2 shaped model, driven through the C ABI.

One `step()` runs, for every block linear (c_attn, attention c_proj, mlp fc, mlp proj) and
the tied LM head, the forward projection Y = X.W^T + b and the backward pass dX = dY.W,
dW = dY^T.X (+ dbias), with every operand quantized to NVFP4 exactly as the reference's
graph does it: four-six for activations (rowwise scale) and weights (tensor scale),
MS-EDEN with counter-RNG stochastic scale rounding for dY, W^T and X^T.  It mirrors the
call sequence of crates/gpt2-nvfp4/src/types/{l2_attention,l3_mlp}/forward.rs,
types/model/final_logits.rs and backward/{linear,mlp/run,attention/*,final_head/run}.rs,
restricted to the projections (attention core, LayerNorm, loss and optimizer are outside
this path; their outputs are stood in for by seeded synthetic tensors).

Tokens are the shardable axis: every rank holds `tokens` rows of X / dY and a full replica
of the weights, and the per-layer dW (+dbias) buckets are summed over ranks with one NCCL
all-reduce each, issued as soon as the layer's backward is enqueued.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import torch

from .sharding import GradBuckets, sync_amax
from . import (EPI_BIAS, EPI_NONE, EPI_RELU2, LinearBackwardModule, LinearBackwardScratch, Nvfp4GemmModule,
               Nvfp4QuantModule, Nvfp4Tensor, SideStream, padded_k, scale_packed_len)

MASK64 = (1 << 64) - 1


class Gpt2Rng:
    """splitmix64 stream handing out the (sign, scale) seeds of each linear
    (crates/gpt2-nvfp4/src/random.rs:1-27)."""

    def __init__(self, seed: int):
        self.state = seed & MASK64

    def next_u64(self) -> int:
        self.state = (self.state + 0x9E3779B97F4A7C15) & MASK64
        z = self.state
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & MASK64
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & MASK64
        return z ^ (z >> 31)

    def next_u32(self) -> int:
        return self.next_u64() & 0xFFFFFFFF


@dataclass(frozen=True)
class ModelShape:
    name: str
    n_layer: int
    d_model: int
    d_mlp: int
    vocab: int

    def linears(self) -> List[Tuple[str, int, int, int]]:
        """(name, in, out, epilogue) of one block, in forward order."""
        d, h = self.d_model, self.d_mlp
        return [("c_attn", d, 3 * d, EPI_BIAS), ("attn_c_proj", d, d, EPI_BIAS), ("mlp_fc", d, h, EPI_RELU2),
                ("mlp_proj", h, d, EPI_BIAS)]

    def macs_per_token(self) -> int:
        per_layer = sum(i * o for _, i, o, _ in self.linears())
        return self.n_layer * per_layer + self.d_model * self.vocab

    def flops_per_token(self) -> int:
        return 6 * self.macs_per_token()  # forward 2, dX 2, dW 2


GPT2_SMALL = ModelShape("gpt2-small-proj-set", 12, 768, 3072, 32000)
GPT2_MEDIUM = ModelShape("gpt2-medium-proj-set", 24, 1024, 4096, 32000)
SHAPES = {"gpt2-small": GPT2_SMALL, "gpt2-medium": GPT2_MEDIUM}


def _randn_bf16(shape, std, seed, device):
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    return (torch.randn(shape, generator=g, device=device, dtype=torch.float32) * std).to(torch.bfloat16)


class _Linear:
    """One projection: master weight, its per-step NVFP4 form, the saved quantized input,
    caller-owned backward scratch and gradient views."""

    def __init__(self, name, in_dim, out_dim, epilogue, tokens, device, seed, has_bias=True, inputs_only=False):
        self.name, self.in_dim, self.out_dim, self.epilogue = name, in_dim, out_dim, epilogue
        self.weight = _randn_bf16((out_dim, in_dim), 0.02, seed, device)
        self.bias = _randn_bf16((out_dim,), 0.02, seed + 1, device).float() if has_bias else None
        self.wq_ready: Optional[torch.cuda.Event] = None
        self.dweight: Optional[torch.Tensor] = None
        self.dbias: Optional[torch.Tensor] = None
        if inputs_only:
            return
        n = out_dim * in_dim
        u8 = dict(dtype=torch.uint8, device=device)
        f32 = dict(dtype=torch.float32, device=device)
        self.wq = Nvfp4Tensor(torch.empty(n // 2, **u8), torch.empty(scale_packed_len(out_dim, in_dim), **u8),
                              torch.empty(1, **f32), out_dim, in_dim, packed=True, rowwise=False)
        self.w_chunk_amax = torch.empty((n + 1023) // 1024, **f32)
        self.w_amax = torch.empty(1, **f32)
        nx = tokens * in_dim
        self.xq = Nvfp4Tensor(torch.empty(nx // 2, **u8), torch.empty(scale_packed_len(tokens, in_dim), **u8),
                              torch.empty(tokens, **f32), tokens, in_dim, packed=True, rowwise=True)
        self.x_amax = torch.empty(tokens, **f32)


class ProjectionSet:
    def __init__(self, shape: ModelShape, tokens: int, device, seed: int = 1234, token_offset: int = 0,
                 process_group=None, grad_dtype: torch.dtype = torch.bfloat16, overlap_weight_quantization: bool = True,
                 fused_mlp: bool = True, total_tokens: int = 0, reproducible_sharding: bool = False,
                 input_seed_offset: Optional[int] = None, inputs_only: bool = False):
        """fused_mlp: the fc projection stores only its pre-activation (plus the row amax of relu(pre)^2 from the
        GEMM epilogue) and the down projection's input quantizer applies relu^2 on load, so the MLP activation is
        never written; False = the fc GEMM writes both tensors and the down projection reads a separate input.
        total_tokens / reproducible_sharding: this rank holds tokens [token_offset, token_offset + tokens) of a
        batch of total_tokens; with reproducible_sharding every amax that feeds a per-tensor scale is
        all-reduced (max) over the ranks in one collective per step and the scale-RNG index spaces are those
        of the unsharded batch, so quantized operands are bit-identical to a single-GPU run.
        inputs_only: allocate only what a step READS (master weights, biases, activations, upstream gradients):
        for callers that hand those tensors to the C++ step driver (`host_step.HostStep`), which owns everything a
        step writes."""
        assert tokens % 128 == 0, "token shards are multiples of 128 rows (scale tiles stay intact)"
        self.shape, self.tokens, self.device = shape, tokens, device
        self.inputs_only = inputs_only
        self.token_offset = token_offset
        self.total_tokens = total_tokens
        self.reproducible = reproducible_sharding
        assert not reproducible_sharding or total_tokens >= token_offset + tokens
        self.fused_mlp = fused_mlp
        self.pg = process_group
        self.grad_dtype = grad_dtype
        self.quant, self.gemm, self.bwd = Nvfp4QuantModule(), Nvfp4GemmModule(), LinearBackwardModule()
        self.seed = seed
        self.rng = Gpt2Rng(seed)
        d, h, v = shape.d_model, shape.d_mlp, shape.vocab
        self.layers: List[List[_Linear]] = []
        for l in range(shape.n_layer):
            self.layers.append([_Linear(n, i, o, e, tokens, device, seed * 1000 + l * 10 + j, inputs_only=inputs_only)
                                for j, (n, i, o, e) in enumerate(shape.linears())])
        self.lm_head = _Linear("lm_head", d, v, EPI_NONE, tokens, device, seed * 1000 + 999, has_bias=False,
                               inputs_only=inputs_only)
        widths_in = sorted({i for _, i, _, _ in shape.linears()} | {d})
        widths_out = sorted({o for _, _, o, _ in shape.linears()} | {v})
        in_seed = token_offset if input_seed_offset is None else input_seed_offset
        # Synthetic stand-ins for the tensors the rest of the model would produce: one activation
        # per input width, one upstream gradient per output width (larger than L2 at bench sizes).
        self.x: Dict[int, torch.Tensor] = {w: _randn_bf16((tokens, w), 1.0, seed + 7 * w + in_seed, device)
                                           for w in widths_in}
        self.dy: Dict[int, torch.Tensor] = {w: _randn_bf16((tokens, w), 1e-3, seed + 11 * w + in_seed, device)
                                            for w in widths_out}
        if inputs_only:
            return
        # one gradient bucket per layer (dW + dbias of its four linears) and one for the LM head
        self.grads = GradBuckets([[(x.out_dim, x.in_dim, True) for x in lin] for lin in self.layers] +
                                 [[(v, d, False)]], device)
        for lin, views in zip(self.layers + [[self.lm_head]], self.grads.views):
            for x, (dw, db) in zip(lin, views):
                x.dweight, x.dbias = dw, db
        self.buckets = self.grads.buffers

        self.y: Dict[int, torch.Tensor] = {w: torch.empty((tokens, w), dtype=torch.bfloat16, device=device)
                                           for w in widths_out}
        self.pre: Dict[int, torch.Tensor] = {h: torch.empty((tokens, h), dtype=torch.bfloat16, device=device)}
        self.pre_row_amax = torch.empty(tokens, dtype=torch.float32, device=device)
        # caller-owned second stream of the linear backward (its two transposers run beside the dY amax pass)
        self.side = SideStream(device)
        n_lin = 4 * shape.n_layer + 1
        self.amax_vec = torch.zeros(2 * n_lin, dtype=torch.float32, device=device)  # [dY amax | decoded X amax]
        self.e_scales = torch.empty(n_lin, dtype=torch.float32, device=device)
        self.dx: Dict[int, torch.Tensor] = {w: torch.empty((tokens, w), dtype=grad_dtype, device=device)
                                            for w in widths_in}
        # backward scratch is shared by all linears of the same (in, out) shape
        self.scratch: Dict[Tuple[int, int], LinearBackwardScratch] = {}
        for _, i, o, _ in shape.linears() + [("lm_head", d, v, EPI_NONE)]:
            if (i, o) not in self.scratch:
                self.scratch[(i, o)] = LinearBackwardScratch(tokens, i, o, device)
        self._weight_stream: Optional[torch.cuda.Stream] = None
        self._weights_quantized = False
        self.overlap_weight_quantization = overlap_weight_quantization
        self.gemm_events: List[Tuple[torch.cuda.Event, torch.cuda.Event, int]] = []
        self.record_gemm_events = False

    # ---- pieces -------------------------------------------------------------------------
    def all_linears(self) -> List[_Linear]:
        return [x for lin in self.layers for x in lin] + [self.lm_head]

    def quantize_weights(self) -> None:
        """Weights are re-quantized from their masters every step (four-six, tensor scale).  The 2 x 49
        launches are tiny (a few microseconds each, a fraction of the SMs), so they go to a side stream in
        the order the forward pass needs them and run in the shadow of the activation quantizers; each
        forward GEMM waits for its own weight's event."""
        if not self.overlap_weight_quantization:
            for lin in self.all_linears():
                self.quant.tensor_amax(lin.weight, lin.w_chunk_amax, lin.w_amax)
                self.quant.quantize_four_six(lin.weight, amax=lin.w_amax, rowwise=False, packed=True, out=lin.wq)
            return
        main = torch.cuda.current_stream()
        if self._weight_stream is None:
            self._weight_stream = torch.cuda.Stream(device=self.device)
            for lin in self.all_linears():
                lin.wq_ready = torch.cuda.Event()
        self._weight_stream.wait_stream(main)  # the previous step has finished with the old NVFP4 weights
        with torch.cuda.stream(self._weight_stream):
            for lin in self.all_linears():
                self.quant.tensor_amax(lin.weight, lin.w_chunk_amax, lin.w_amax)
                self.quant.quantize_four_six(lin.weight, amax=lin.w_amax, rowwise=False, packed=True, out=lin.wq)
                lin.wq_ready.record(self._weight_stream)

    def _forward_linear(self, lin: _Linear) -> None:
        if self.fused_mlp and lin.name == "mlp_proj":
            # the MLP activation relu(pre)^2 is computed on load from the fc projection's pre-activation;
            # its row amax came out of that GEMM's epilogue
            self.quant.quantize_relu2_four_six_rowwise(self.pre[lin.in_dim], row_amax=self.pre_row_amax, packed=True,
                                                       out=lin.xq, decoded_amax=True)
        else:
            # row amax fused; the decoded amax rides along so that backward need not re-read X for it
            self.quant.quantize_four_six(self.x[lin.in_dim], rowwise=True, packed=True, out=lin.xq, decoded_amax=True)
        if lin.wq_ready is not None:
            torch.cuda.current_stream().wait_event(lin.wq_ready)
        flops = 2 * self.tokens * lin.in_dim * lin.out_dim
        if self.fused_mlp and lin.epilogue == EPI_RELU2:
            self._timed_gemm(lambda: self.gemm.gemm(lin.xq, lin.wq, bias=lin.bias, epilogue=EPI_BIAS,
                                                    out=self.pre[lin.out_dim], relu2_row_amax=self.pre_row_amax), flops)
            return
        aux = self.pre[lin.out_dim] if lin.epilogue == EPI_RELU2 else None
        self._timed_gemm(lambda: self.gemm.gemm(lin.xq, lin.wq, bias=lin.bias, epilogue=lin.epilogue,
                                                out=self.y[lin.out_dim], aux=aux), flops)

    def _backward_order(self) -> List[_Linear]:
        order = [self.lm_head]
        for l in range(self.shape.n_layer - 1, -1, -1):
            order += list(reversed(self.layers[l]))
        return order

    def _sync_scales(self) -> None:
        """Reproducible sharding: the amax of every dY and of every decoded X of this step as ONE f32 vector,
        all-reduced (max) over the ranks; the dY scales are derived from the reduced values."""
        order = self._backward_order()
        n = len(order)
        for i, lin in enumerate(order):
            self.quant.tensor_amax(self.dy[lin.out_dim], out=self.amax_vec[i:i + 1],
                                   chunk_amax=self.scratch[(lin.in_dim, lin.out_dim)].e_h["chunk_amax"])
            self.amax_vec[n + i:n + i + 1].copy_(lin.xq.decoded_amax)
        sync_amax(self.amax_vec, self.pg)
        for i in range(n):
            self.quant.quartet_backward_ms_eden_global_scale_from_chunks(self.amax_vec[i:i + 1], 1,
                                                                         out=self.e_scales[i:i + 1])

    def _backward_linear(self, lin: _Linear, index: int = 0) -> None:
        sign_seed, scale_seed = self.rng.next_u32(), self.rng.next_u32()
        extra = {}
        if self.reproducible:
            n = 4 * self.shape.n_layer + 1
            extra = dict(total_token_count=self.total_tokens, e_global_scale=self.e_scales[index:index + 1],
                         x_decoded_amax=self.amax_vec[n + index:n + index + 1])
        self.bwd.backward_ms_eden(e=self.dy[lin.out_dim], weight=lin.wq, input=lin.xq,
                                  scratch=self.scratch[(lin.in_dim, lin.out_dim)], sign_seed=sign_seed,
                                  scale_seed=scale_seed, want_dbias=lin.dbias is not None,
                                  dinput=self.dx[lin.in_dim], dweight=lin.dweight, dbias=lin.dbias,
                                  token_offset=self.token_offset, side=self.side, **extra)

    def _timed_gemm(self, fn, flops: int) -> None:
        if self.record_gemm_events:
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            self.gemm_events.append((a, b, flops))
        else:
            fn()

    def _reduce(self, layer: int) -> None:
        if self.pg is not None:
            self.grads.reduce_async(layer, self.pg)

    # ---- one step -----------------------------------------------------------------------
    def forward(self) -> None:
        for lin in self.layers:
            for x in lin:
                self._forward_linear(x)
        self._forward_linear(self.lm_head)

    def backward(self) -> None:
        if self.reproducible:
            self._sync_scales()
        self._backward_linear(self.lm_head, 0)
        self._reduce(self.shape.n_layer)
        index = 1
        for l in range(self.shape.n_layer - 1, -1, -1):
            for x in reversed(self.layers[l]):
                self._backward_linear(x, index)
                index += 1
            self._reduce(l)
        self.grads.wait()

    def step(self, weights_changed: bool = True) -> None:
        """One forward + backward pass over this rank's tokens.  `weights_changed=False` (the second and later
        micro-steps of a gradient accumulation, where no optimizer update happened in between) reuses the
        packed NVFP4 weights of the previous step instead of re-quantizing the masters; W^T cannot be reused
        the same way because its MS-EDEN form is drawn with fresh seeds in every linear backward."""
        if weights_changed or not self._weights_quantized:
            self.quantize_weights()
            self._weights_quantized = True
        self.forward()
        self.backward()

    def capture_step(self) -> "torch.cuda.CUDAGraph":
        """One step captured in a CUDA graph (single rank; call after at least one eager step so that
        one-time set-up is done).  The library allocates nothing and never synchronises inside a step,
        and tensor maps travel as kernel parameters, so the whole step is capturable; the MS-EDEN seeds
        drawn during capture are baked into the graph."""
        assert self.pg is None, "graph capture is offered for the single-rank step only"
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            self.step()
        return graph

    def flops_per_step(self) -> int:
        return self.shape.flops_per_token() * self.tokens

    def result_digest(self) -> torch.Tensor:
        """A small device vector summarising the step's outputs (read back by the e2e timing)."""
        return torch.stack([b.abs().sum() for b in self.buckets])
