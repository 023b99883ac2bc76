"""One decode step of a pre-norm decoder stack with fp8-e4m3 linears -- the shape of xn-moshi's
BatchedTransformerLayer (xn-moshi/src/batched_transformer.rs:92-199, 246-268) with the gated FFN of
xn-moshi/src/transformer.rs:234-247, restricted to what the benchmark's decoder configuration lists:
RMSNorm -> fused qkv projection -> KV append -> attention over a (streams, heads, context, 128) bf16
cache -> output projection -> residual -> RMSNorm -> gated SiLU FFN -> residual.  No rope (the
configuration does not list it).  T = 1 token per stream per step; streams are independent, which is
what lets them be sharded over GPUs with no communication.

Every operation is a call into libxn_mm.so on the current torch stream, so a step can be captured in
a CUDA graph.  Buffers are allocated once in the constructor.
"""
from __future__ import annotations

import math

import torch

from ._lib import BF16, check, lib


class DecoderStack:
    def __init__(self, n_layers: int, d_model: int, n_heads: int, ffn_hidden: int, streams: int, context: int,
                 device, eps: float = 1e-5, seed: int = 4, variant: int = 0, kv_init: str = "normal",
                 attention: str = "separate"):
        """attention: how a layer's cache append, attention, merge of the context slices and e4m3 split are launched.
        "separate" = xn_mm_kv_append2 + xn_mm_decode_attention_split_e4m3 (three launches; the fastest at 32 streams x
        3000 tokens), "fused" = xn_mm_decode_attention_append_e4m3 (one or two launches, the library decides where the
        merge runs), "fused_one_launch" = the same with the merge forced into the attention kernel.  All three give
        identical results."""
        assert d_model == n_heads * 128, "head_dim is 128"
        assert attention in ("separate", "fused", "fused_one_launch")
        self.attention = attention
        self.L, self.d, self.H, self.hid, self.B, self.ctx = n_layers, d_model, n_heads, ffn_hidden, streams, context
        self.eps, self.variant, self.dev = eps, variant, device
        g = torch.Generator(device=device).manual_seed(seed)
        from .ops import quantize_weights_fp8

        def qlin(n, k):
            w = torch.randn(n, k, generator=g, device=device) * 0.02
            q = quantize_weights_fp8(w)
            del w
            return q

        self.layers = []
        for _ in range(n_layers):
            lay = {
                "norm1": torch.ones(d_model, device=device, dtype=torch.bfloat16),
                "norm2": torch.ones(d_model, device=device, dtype=torch.bfloat16),
                "in_proj": qlin(3 * d_model, d_model),
                "out_proj": qlin(d_model, d_model),
                "linear_in": qlin(2 * ffn_hidden, d_model),
                "linear_out": qlin(d_model, ffn_hidden),
            }
            shape = (streams, n_heads, context, 128)
            if kv_init == "normal":
                lay["k"] = torch.randn(shape, generator=g, device=device, dtype=torch.bfloat16)
                lay["v"] = torch.randn(shape, generator=g, device=device, dtype=torch.bfloat16)
            else:
                lay["k"] = torch.zeros(shape, device=device, dtype=torch.bfloat16)
                lay["v"] = torch.zeros(shape, device=device, dtype=torch.bfloat16)
            self.layers.append(lay)
        B, d, hid = streams, d_model, ffn_hidden
        kmax = max(d, hid)
        u8 = dict(dtype=torch.uint8, device=device)
        bf = dict(dtype=torch.bfloat16, device=device)
        self.hi, self.lo = torch.empty(B * kmax, **u8), torch.empty(B * kmax, **u8)
        self.xs = torch.empty(B, dtype=torch.float32, device=device)
        self.qkv = torch.empty(B, 3 * d, **bf)
        self.attn = torch.empty(B, d, **bf)
        # (maximum, sum, output) records of the context slices of the attention
        self.attn_ws_bytes = int(lib().xn_mm_decode_attention_append_workspace_bytes(B, n_heads, context))
        self.attn_ws = torch.empty(self.attn_ws_bytes, dtype=torch.uint8, device=device)
        self.proj = torch.empty(B, d, **bf)
        self.h = torch.empty(B, 2 * hid, **bf)
        self.x_mid = torch.empty(B, d, **bf)
        self.x_out = torch.empty(B, d, **bf)
        self.pos = torch.full((B,), context - 1, dtype=torch.int64, device=device)
        self.mask = None  # optional f32 [B, context] additive mask

    # -- helpers -------------------------------------------------------------------------------
    def _s(self):
        return torch.cuda.current_stream().cuda_stream

    def _linear(self, y, wq_ws, m, n, k):
        wq, ws = wq_ws
        check(lib().xn_mm_linear_fp8_pieces(y.data_ptr(), self.hi.data_ptr(),
                                            self.lo.data_ptr() if self.variant == 0 else None, self.xs.data_ptr(),
                                            wq.data_ptr(), ws.data_ptr(), m, n, k, self._s()))

    def _lo(self):
        return self.lo.data_ptr() if self.variant == 0 else None

    def step(self, x: torch.Tensor) -> torch.Tensor:
        """x: [streams, d_model] bf16 (the embedded token of every stream). Returns the stack's output."""
        L, B, d, H, hid, ctx = lib(), self.B, self.d, self.H, self.hid, self.ctx
        s = self._s()
        cur = x
        for li, lay in enumerate(self.layers):
            if li == 0:  # later layers get their pieces from the fused add + norm that ends the previous layer
                check(L.xn_mm_rms_norm_split_e4m3(self.hi.data_ptr(), self._lo(), self.xs.data_ptr(), None, cur.data_ptr(),
                                                  lay["norm1"].data_ptr(), BF16, B, d, self.eps, s))
            self._linear(self.qkv, lay["in_proj"], B, 3 * d, d)
            q, kn, vn = self.qkv.data_ptr(), self.qkv.data_ptr() + 2 * d, self.qkv.data_ptr() + 4 * d
            if self.attention == "separate":
                check(L.xn_mm_kv_append2(BF16, lay["k"].data_ptr(), lay["v"].data_ptr(), kn, vn, 3 * d, self.pos.data_ptr(), B, H,
                                         ctx, 128, s))
                # attention over the cache; the merge of the context slices also writes the e4m3 pieces of the output row
                check(L.xn_mm_decode_attention_split_e4m3(self.hi.data_ptr(), self._lo(), self.xs.data_ptr(),
                                                          self.attn.data_ptr(), q, 3 * d, lay["k"].data_ptr(),
                                                          lay["v"].data_ptr(),
                                                          self.mask.data_ptr() if self.mask is not None else None, B, H, ctx,
                                                          128, 1.0 / math.sqrt(128.0), self.attn_ws.data_ptr(),
                                                          self.attn_ws_bytes, s))
            else:
                # append the new key / value rows, attend over the cache, merge the context slices and write the e4m3
                # pieces of the output row
                check(L.xn_mm_decode_attention_append_e4m3(self.hi.data_ptr(), self._lo(), self.xs.data_ptr(),
                                                           self.attn.data_ptr(), q, kn, vn, 3 * d, lay["k"].data_ptr(),
                                                           lay["v"].data_ptr(), self.pos.data_ptr(),
                                                           self.mask.data_ptr() if self.mask is not None else None, B, H, ctx,
                                                           128, 1.0 / math.sqrt(128.0),
                                                           1 if self.attention == "fused_one_launch" else 0,
                                                           self.attn_ws.data_ptr(), self.attn_ws_bytes, s))
            self._linear(self.proj, lay["out_proj"], B, d, d)
            check(L.xn_mm_add_rms_norm_split_e4m3(self.hi.data_ptr(), self._lo(), self.xs.data_ptr(), self.x_mid.data_ptr(),
                                                  cur.data_ptr(), self.proj.data_ptr(), lay["norm2"].data_ptr(), BF16, B, d,
                                                  self.eps, s))
            self._linear(self.h, lay["linear_in"], B, 2 * hid, d)
            check(L.xn_mm_silu_mul_split_e4m3(self.hi.data_ptr(), self._lo(), self.xs.data_ptr(), self.h.data_ptr(), BF16,
                                              B, hid, s))
            self._linear(self.proj, lay["linear_out"], B, d, hid)
            if li + 1 < len(self.layers):  # x_out = x_mid + proj, pieces of the next layer's norm1(x_out)
                check(L.xn_mm_add_rms_norm_split_e4m3(self.hi.data_ptr(), self._lo(), self.xs.data_ptr(),
                                                      self.x_out.data_ptr(), self.x_mid.data_ptr(), self.proj.data_ptr(),
                                                      self.layers[li + 1]["norm1"].data_ptr(), BF16, B, d, self.eps, s))
            else:
                check(L.xn_mm_add(BF16, self.x_out.data_ptr(), self.x_mid.data_ptr(), self.proj.data_ptr(), B * d, s))
            cur = self.x_out
        return self.x_out

    def bytes_per_step(self) -> dict:
        d, hid, B, ctx, H = self.d, self.hid, self.B, self.ctx, self.H
        w = self.L * (3 * d * d + d * d + 2 * hid * d + d * hid + 4 * (3 * d + d + 2 * hid + d))
        kv = self.L * 2 * B * H * ctx * 128 * 2
        return {"weights": w, "kv": kv, "total": w + kv}

    def launches_per_step(self) -> int:
        # per layer: in_proj, cache append + attention + merge of the context slices with the e4m3 split (three launches,
        # two or one, see `attention`), out_proj, add+norm, linear_in, silu*mul, linear_out, add+norm (plain add after the last layer); one norm
        # up front
        per_layer = 10 if self.attention == "separate" else (8 if self._merge_in_kernel() else 9)
        return self.L * per_layer + 1

    def _merge_in_kernel(self) -> bool:
        """The library's policy (xn_mm_decode_attention_append_e4m3): the merge of the context slices runs inside the
        attention kernel when a resident slot sees at most two CTAs, otherwise as its own launch."""
        if self.attention == "fused_one_launch":
            return True
        ctas = self.attn_ws_bytes // (130 * 4)  # one 130-float record per (stream, head, slice)
        sms = torch.cuda.get_device_properties(self.dev).multi_processor_count
        return ctas <= sms * 5 * 2
