"""TEST INFRASTRUCTURE - the checker at the benchmark configurations' real sizes.

oracle/oracle.c walks every weight row element by element in double precision: exact, and far too slow for a 2048-token prompt on an 8B-shaped model.
This module restates the same decoder (the reference test's `Reference::step`, tests/unit/test_metal_llama_decoder.cpp:114-161, applied to a whole chunk
of positions) with one layer's weights in memory at a time: the layer's matrices are dequantized by oracle.c's block formulas (oracle_dequantize, the
bit-exact ones) and the arithmetic runs as float64 torch matmuls on whatever device the caller names. With `round_operands` the chunk's projections see
their operands rounded to f16 exactly where oracle.c's variant of that name rounds them (the reference's prefill tiles, llama_kernels.h:186-199, 372, 660,
717); keys and values are rounded to f16 into the cache in both modes.

It is validated against oracle.c itself (tests/test_oracle.py, CPU, small models). On a CUDA device the matmuls are torch's float64 GEMMs: library code
used as a calculator by the checker, never by the product, and only in tests.
"""
from __future__ import annotations

import ctypes as C
import math

import numpy as np
import torch

from dooms_b200 import _lib as L

from . import binding as ob


def _dequantized(ref, device) -> torch.Tensor:
    """A weight tensor dequantized with the checker's block formulas, f32 [rows][cols] (a matrix of whole rows is one long run of blocks, which is what
    oracle_dequantize walks)."""
    n = ref.rows * ref.cols
    nbytes = n // L.BLOCK_ELEMS[ref.dtype] * L.BLOCK_BYTES[ref.dtype]
    raw = np.ctypeslib.as_array(C.cast(ref.data, C.POINTER(C.c_uint8)), shape=(nbytes,))
    out = np.empty(n, dtype=np.float32)
    ob.oracle().oracle_dequantize(ref.dtype, raw.ctypes.data, n, out.ctypes.data)
    return torch.from_numpy(out.reshape(ref.rows, ref.cols)).to(device=device)


def _half(t: torch.Tensor) -> torch.Tensor:
    return t.to(torch.float16).to(t.dtype)


class StreamingOracle:
    """eval_tokens / eval_embeddings over a GGUF file, one layer resident at a time. `taps`, when given, collects sampled rows of every layer's output
    (the residual stream after the layer) for comparison with a device-side copy."""

    def __init__(self, path: str, n_ctx: int, device: str = "cpu", round_operands: bool = False, keep_weights: bool = False):
        """keep_weights: the dequantized tensors stay on the device as f32 (exactly the dequantized values) after their first use, so that single positions
        after a prompt do not dequantize the whole model again; needs 4 bytes per weight of device memory."""
        self.cfg, self.w, self._keep = ob.model_structs(path, n_ctx)
        self.device = torch.device(device)
        self.round_operands = round_operands
        self._kept: dict[int, torch.Tensor] | None = {} if keep_weights else None
        c = self.cfg
        kv = c.n_head_kv * c.head_dim
        self.kc = torch.zeros(c.n_layer, n_ctx, kv, dtype=torch.float64, device=self.device)
        self.vc = torch.zeros_like(self.kc)
        self.pos = 0
        i = torch.arange(c.head_dim // 2, dtype=torch.float64, device=self.device)
        self.inv_freq = torch.pow(torch.tensor(float(c.rope_base), dtype=torch.float64, device=self.device), -2.0 * i / c.head_dim)
        self.layer_rows: dict[int, torch.Tensor] = {}

    def reset(self):
        self.pos = 0

    def _tensor(self, ref) -> torch.Tensor:
        if self._kept is None:
            return _dequantized(ref, self.device).double()
        t = self._kept.get(ref.data)
        if t is None:
            t = self._kept[ref.data] = _dequantized(ref, self.device)
        return t.double()

    def _rms(self, x, gamma, round_ops):
        inv = torch.rsqrt((x * x).mean(dim=1, keepdim=True) + float(self.cfg.rms_eps))
        y = x * inv * gamma
        return _half(y.float()).double() if round_ops else y

    def _rope(self, v, positions):
        """v: [M][heads][head_dim]; rotates in place the pairs (2i, 2i+1) or (i, i + head_dim / 2)."""
        hd = self.cfg.head_dim
        th = positions.double()[:, None] * self.inv_freq[None, :]
        cos, sin = torch.cos(th)[:, None, :], torch.sin(th)[:, None, :]
        if self.cfg.rope_neox:
            a, b = v[..., : hd // 2].clone(), v[..., hd // 2:].clone()
            v[..., : hd // 2] = a * cos - b * sin
            v[..., hd // 2:] = a * sin + b * cos
        else:
            a, b = v[..., 0::2].clone(), v[..., 1::2].clone()
            v[..., 0::2] = a * cos - b * sin
            v[..., 1::2] = a * sin + b * cos
        return v

    def embeddings(self, tokens) -> torch.Tensor:
        c = self.cfg
        ref = self.w.token_embd
        rb = c.n_embd // L.BLOCK_ELEMS[ref.dtype] * L.BLOCK_BYTES[ref.dtype]
        raw = np.ctypeslib.as_array(C.cast(ref.data, C.POINTER(C.c_uint8)), shape=(ref.rows * rb,))
        rows = np.stack([ob.dequantize(ref.dtype, raw[int(t) * rb:(int(t) + 1) * rb], c.n_embd) for t in tokens])
        return torch.from_numpy(rows)

    def eval_tokens(self, tokens, tap_rows=None) -> np.ndarray:
        return self.eval_embeddings(self.embeddings(tokens), tap_rows)

    def eval_embeddings(self, emb, tap_rows=None) -> np.ndarray:
        """Appends the rows of emb; the last row's logits as float64. tap_rows: indices of rows whose value after every layer is kept in layer_rows[l]."""
        c = self.cfg
        dev = self.device
        x = torch.as_tensor(np.asarray(emb, dtype=np.float32)).to(dev).double()
        M = x.shape[0]
        assert self.pos + M <= self.kc.shape[1]
        E, hd, nh, nkv = c.n_embd, c.head_dim, c.n_head, c.n_head_kv
        Q, KV = nh * hd, nkv * hd
        ro = self.round_operands and M > 1
        rw = (lambda w: _half(w.float()).double()) if ro else (lambda w: w)
        positions = torch.arange(self.pos, self.pos + M, device=dev)
        self.layer_rows = {}
        for l in range(c.n_layer):
            lw = self.w.layers[l]
            xn = self._rms(x, self._tensor(lw.attn_norm).reshape(-1), ro)
            if lw.attn_qkv.data:
                qkv = xn @ rw(self._tensor(lw.attn_qkv)).T
            else:
                qkv = torch.cat([xn @ rw(self._tensor(r)).T for r in (lw.attn_q, lw.attn_k, lw.attn_v)], dim=1)
            if lw.attn_qkv_bias.data:
                qkv = qkv + self._tensor(lw.attn_qkv_bias).reshape(-1)
            elif lw.attn_q_bias.data:
                qkv = qkv + torch.cat([self._tensor(r).reshape(-1) for r in (lw.attn_q_bias, lw.attn_k_bias, lw.attn_v_bias)])
            q = self._rope(qkv[:, :Q].reshape(M, nh, hd).clone(), positions)
            k = self._rope(qkv[:, Q:Q + KV].reshape(M, nkv, hd).clone(), positions)
            v = qkv[:, Q + KV:].reshape(M, nkv, hd)
            self.kc[l, self.pos:self.pos + M] = _half(k.reshape(M, KV).float()).double()
            self.vc[l, self.pos:self.pos + M] = _half(v.reshape(M, KV).float()).double()
            n = self.pos + M
            keys = self.kc[l, :n].reshape(n, nkv, hd)
            vals = self.vc[l, :n].reshape(n, nkv, hd)
            att = torch.empty(M, nh, hd, dtype=torch.float64, device=dev)
            g = nh // nkv
            causal = torch.arange(n, device=dev)[None, :] <= positions[:, None]          # [M][n]
            if ro:          # the prefill tiles hold the rotated query as f16 (attention_prefill, llama_kernels.h:660)
                q = _half(q.float()).double()
            for h in range(nh):
                s = (q[:, h, :] @ keys[:, h // g, :].T) / math.sqrt(hd)
                s = s.masked_fill(~causal, float("-inf"))
                if ro:      # ... and the probabilities as f16 relative to the row maximum; the normalizing sum adds the unrounded exponentials (:708-713)
                    e = torch.exp(s - s.max(dim=1, keepdim=True).values)
                    att[:, h, :] = (_half(e.float()).double() @ vals[:, h // g, :]) / e.sum(dim=1, keepdim=True)
                else:
                    att[:, h, :] = torch.softmax(s, dim=1) @ vals[:, h // g, :]
            att = att.reshape(M, Q)
            if ro:
                att = _half(att.float()).double()
            x = x + att @ rw(self._tensor(lw.attn_output)).T
            xn = self._rms(x, self._tensor(lw.ffn_norm).reshape(-1), ro)
            gate = xn @ rw(self._tensor(lw.ffn_gate)).T
            up = xn @ rw(self._tensor(lw.ffn_up)).T
            hid = gate / (1 + torch.exp(-gate)) * up
            del gate, up
            if ro:
                hid = _half(hid.float()).double()
            x = x + hid @ rw(self._tensor(lw.ffn_down)).T
            del hid
            if tap_rows is not None:
                self.layer_rows[l] = x[list(tap_rows)].cpu().numpy()
        last = self._rms(x[M - 1:M], self._tensor(self.w.output_norm).reshape(-1), False)
        logits = last @ self._tensor(self.w.output).T
        self.pos += M
        return logits.reshape(-1).cpu().numpy()
