"""BERT encoder runner: the exported ONNX subgraph of `transformers` BertLayer executed through the C ABI.

This is the caller side of the hot path for the BERT configurations: what DaCeML's
`DaceModule(BertLayer)` runs after node expansion (daceml/pytorch/module.py:212-295 builds it,
tests/pytorch/test_bert_encoder.py:10-50 exercises it), with the elementwise chains folded into
the contraction epilogues where the graph allows it:

    MatMul(x, Transpose(W)) + Add(bias)                      -> gemm, trans_b, EPI_BIAS
    ... + Add(residual)                                      -> EPI_BIAS_RESIDUAL
    ... + Div/Erf/Add/Mul/Mul (Gelu)                         -> EPI_BIAS_GELU
    MatMul(q, k^T), Mul(1/sqrt(d)), Softmax, MatMul(p, v)    -> one fused attention kernel (TF32 mode,
                                                                head_dim 64, seq % 32 == 0); otherwise:
    MatMul(q, k^T) + Mul(1/sqrt(d))                          -> batched gemm, EPI_SCALE
    Reshape/Transpose [0,2,1,3] either side of attention     -> strided batch addressing (no copy)
    ReduceMean..Add (9 nodes)                                -> layernorm

Torch provides device buffers, streams and (for several GPUs) the process group; all arithmetic
is in libb200ops.
"""
import math

import torch

from . import ops
from ._lib import EPI_BIAS, EPI_BIAS_GELU, EPI_BIAS_RESIDUAL, EPI_SCALE


def synthetic_layer_params(hidden, ffn, seed, std=0.02):
    """Random-init weights of one encoder layer for benchmarks: matrices ~ N(0, std^2) from a seeded CPU
    generator (the same values on every rank that uses the same seed), biases 0, LayerNorm gamma 1 / beta 0."""
    g = torch.Generator().manual_seed(int(seed))
    p = {}
    for key, shape in (("wq", (hidden, hidden)), ("wk", (hidden, hidden)), ("wv", (hidden, hidden)),
                       ("wo", (hidden, hidden)), ("wi", (ffn, hidden)), ("wo2", (hidden, ffn))):
        p[key] = torch.randn(*shape, generator=g, dtype=torch.float32) * std
    for key, n in (("bq", hidden), ("bk", hidden), ("bv", hidden), ("bo", hidden), ("bi", ffn), ("bo2", hidden),
                   ("ln1_b", hidden), ("ln2_b", hidden)):
        p[key] = torch.zeros(n, dtype=torch.float32)
    p["ln1_g"] = torch.ones(hidden, dtype=torch.float32)
    p["ln2_g"] = torch.ones(hidden, dtype=torch.float32)
    return p


class BertEncoderB200:
    """N identical-shape BERT encoder layers on one GPU.

    `layers` is a list of dicts with keys wq,bq,wk,bk,wv,bv,wo,bo,ln1_g,ln1_b,wi,bi,wo2,bo2,
    ln2_g,ln2_b (Linear weights in torch layout [out, in]). The batch is processed in micro-batches
    of `micro_batch` sequences so that the materialised [b, heads, S, S] score tensor stays bounded.
    """

    def __init__(self, layers, heads, eps=1e-12, device="cuda:0", math_mode="fp32x3", micro_batch=128,
                 fused_attention=True):
        self.device = torch.device(device)
        self.heads = heads
        self.eps = float(eps)
        self.math_mode = math_mode
        self.micro_batch = int(micro_batch)
        self.fused_attention = bool(fused_attention)
        self.hidden = layers[0]["wq"].shape[0]
        self.ffn = layers[0]["wi"].shape[0]
        if self.hidden % heads:
            raise ValueError("hidden size must be a multiple of the head count")
        self.head_dim = self.hidden // heads
        dev = lambda t: t.detach().to(self.device, torch.float32).contiguous()  # noqa: E731
        self.layers = []
        for p in layers:
            self.layers.append(dict(
                # the three projections share their input: one GEMM against the stacked weight rows
                wqkv=dev(torch.cat([p["wq"], p["wk"], p["wv"]], 0)), bqkv=dev(torch.cat([p["bq"], p["bk"], p["bv"]], 0)),
                wo=dev(p["wo"]), bo=dev(p["bo"]), ln1_g=dev(p["ln1_g"]), ln1_b=dev(p["ln1_b"]),
                wi=dev(p["wi"]), bi=dev(p["bi"]), wo2=dev(p["wo2"]), bo2=dev(p["bo2"]),
                ln2_g=dev(p["ln2_g"]), ln2_b=dev(p["ln2_b"])))
        self._buf_key = None
        self._buf = None
        self._io = None            # staging buffers and copy streams of forward_host
        self.launches = 0          # C-ABI kernel launches issued so far
        self.timeline = None       # when a list: (kind, flops, bytes, start_event, end_event) per launch

    # -- scratch --------------------------------------------------------------------------------
    def _buffers(self, mb, seq):
        key = (mb, seq)
        if self._buf_key != key:
            h, f, nh = self.hidden, self.ffn, self.heads
            e = lambda *s: torch.empty(s, device=self.device, dtype=torch.float32)  # noqa: E731
            self._buf = dict(qkv=e(mb, seq, 3 * h), ctx=e(mb, seq, h), attn=e(mb, seq, h), h1=e(mb, seq, h),
                             inter=e(mb, seq, f), out=e(mb, seq, h), ping=e(mb, seq, h), pong=e(mb, seq, h))
            self._buf_key = key
        return self._buf

    def release_buffers(self):
        """Drop the scratch and staging buffers (they are re-created on the next call)."""
        self._buf_key = self._buf = self._io = None

    def _score_buffers(self, mb, seq):
        """[mb, heads, S, S] scores and probabilities, only needed by the unfused attention path."""
        buf = self._buf
        if "scores" not in buf:
            buf["scores"] = torch.empty(mb, self.heads, seq, seq, device=self.device, dtype=torch.float32)
            buf["probs"] = torch.empty_like(buf["scores"])
        return buf["scores"], buf["probs"]

    def _timed(self, kind, flops, nbytes, fn):
        self.launches += 1
        if self.timeline is None:
            r = fn()
            if r is False:
                self.launches -= 1
            return r
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        r = fn()
        e.record()
        if r is False:  # the op declined (fused attention not applicable): nothing was launched
            self.launches -= 1
            return r
        self.timeline.append((kind, flops, nbytes, s, e))
        return r

    # -- one layer on one micro-batch -------------------------------------------------------------
    def _layer(self, x, y, w, buf, b, seq):
        h, f, nh, d, mm = self.hidden, self.ffn, self.heads, self.head_dim, self.math_mode
        t = b * seq
        x2 = x.view(t, h)
        qkv, ctx = buf["qkv"][:b], buf["ctx"][:b]
        attn, h1, inter, out = buf["attn"][:b], buf["h1"][:b], buf["inter"][:b], buf["out"][:b]

        self._timed("gemm", 2 * t * 3 * h * h, 0, lambda: ops.matmul(
            x2, w["wqkv"], out=qkv.view(t, 3 * h), trans_b=True, epilogue=EPI_BIAS, bias=w["bqkv"], math_mode=mm))
        # MatMul -> Mul -> Softmax -> MatMul as one kernel when the fused attention covers the case
        q4 = qkv.view(b, seq, 3 * nh, d)
        fused = self.fused_attention and self._timed(
            "attention", 4 * b * nh * seq * seq * d, 16 * t * h,
            lambda: ops.attention_views(q4[:, :, :nh], q4[:, :, nh:2 * nh], q4[:, :, 2 * nh:], ctx.view(b, seq, nh, d),
                                        1.0 / math.sqrt(d), math_mode=mm))
        if fused is False:
            scores, probs = self._score_buffers(buf["qkv"].shape[0], seq)
            self._attention_unfused(qkv, scores[:b], probs[:b], ctx, b, seq)
        self._timed("gemm", 2 * t * h * h, 0, lambda: ops.matmul(
            ctx.view(t, h), w["wo"], out=attn.view(t, h), trans_b=True, epilogue=EPI_BIAS_RESIDUAL, bias=w["bo"],
            residual=x2, math_mode=mm))
        self._timed("layernorm", 0, 8 * t * h, lambda: ops.layernorm(attn, w["ln1_g"], w["ln1_b"], self.eps, out=h1))
        self._timed("gemm", 2 * t * f * h, 0, lambda: ops.matmul(
            h1.view(t, h), w["wi"], out=inter.view(t, f), trans_b=True, epilogue=EPI_BIAS_GELU, bias=w["bi"],
            math_mode=mm))
        self._timed("gemm", 2 * t * f * h, 0, lambda: ops.matmul(
            inter.view(t, f), w["wo2"], out=out.view(t, h), trans_b=True, epilogue=EPI_BIAS_RESIDUAL, bias=w["bo2"],
            residual=h1.view(t, h), math_mode=mm))
        self._timed("layernorm", 0, 8 * t * h, lambda: ops.layernorm(out, w["ln2_g"], w["ln2_b"], self.eps, out=y))
        return y

    def _attention_unfused(self, qkv, scores, probs, ctx, b, seq):
        h, nh, d, mm = self.hidden, self.heads, self.head_dim, self.math_mode
        t = b * seq
        # scores[b,n] = q[b,:,n,:] @ k[b,:,n,:]^T * 1/sqrt(d), heads addressed inside qkv
        self._timed("gemm_qk", 2 * b * nh * seq * seq * d, 4 * (2 * t * h + b * nh * seq * seq), lambda: ops.gemm_raw(
            qkv, qkv[..., h:], scores, batch_outer=b, batch_inner=nh, M=seq, N=seq, K=d, lda=3 * h, ldb=3 * h,
            ldy=seq, a_strides=(seq * 3 * h, d), b_strides=(seq * 3 * h, d), y_strides=(nh * seq * seq, seq * seq),
            trans_b=True, epilogue=EPI_SCALE, scale=1.0 / math.sqrt(d), math_mode=mm))
        self._timed("softmax", 0, 8 * b * nh * seq * seq, lambda: ops.softmax(scores, 3, out=probs))
        # ctx[b,:,n,:] = probs[b,n] @ v[b,:,n,:]; written straight into [b, S, hidden]
        self._timed("gemm_pv", 2 * b * nh * seq * seq * d, 4 * (2 * t * h + b * nh * seq * seq), lambda: ops.gemm_raw(
            probs, qkv[..., 2 * h:], ctx, batch_outer=b, batch_inner=nh, M=seq, N=d, K=seq, lda=seq, ldb=3 * h,
            ldy=h, a_strides=(nh * seq * seq, seq * seq), b_strides=(seq * 3 * h, d), y_strides=(seq * h, d),
            trans_b=False, math_mode=mm))

    # -- whole encoder ------------------------------------------------------------------------------
    def device_chunks(self, bsz, tail_chunks=1):
        """[(lo, n), ...]: the pieces of the batch in the order forward_device completes them -- one per
        micro-batch, the last micro-batch's final layer cut into `tail_chunks` pieces (so that whatever consumes
        finished pieces, e.g. the output all-gather, has only a small last piece left when the forward ends)."""
        mb = min(self.micro_batch, max(bsz, 1))
        out = []
        for b0 in range(0, bsz, mb):
            b = min(mb, bsz - b0)
            if b0 + b >= bsz and tail_chunks > 1 and b >= 8 * tail_chunks:
                cb = -(-b // tail_chunks)
                out.extend((b0 + c0, min(cb, b - c0)) for c0 in range(0, b, cb))
            else:
                out.append((b0, b))
        return out

    def forward_device(self, x, out=None, tail_chunks=1, on_chunk=None):
        """x: [B, S, hidden] fp32 on this encoder's device. Returns [B, S, hidden] on the device.
        `on_chunk(lo, n)` is called (on the host, in stream order) after the launches that complete samples
        [lo, lo+n) of `out`; the pieces are those of device_chunks(B, tail_chunks)."""
        if x.device != self.device or x.dtype != torch.float32 or x.dim() != 3 or x.shape[2] != self.hidden:
            raise ValueError("expected a float32 [B, S, %d] tensor on %s" % (self.hidden, self.device))
        x = x.contiguous()
        bsz, seq, _ = x.shape
        if out is None:
            out = torch.empty_like(x)
        mb = min(self.micro_batch, max(bsz, 1))
        buf = self._buffers(mb, seq)
        pieces = self.device_chunks(bsz, tail_chunks)
        for b0 in range(0, bsz, mb):
            b = min(mb, bsz - b0)
            cur = x[b0:b0 + b]
            mine = [(lo, n) for lo, n in pieces if b0 <= lo < b0 + b]
            for li, w in enumerate(self.layers):
                last = li + 1 == len(self.layers)
                if last:
                    for lo, n in mine:
                        self._layer(cur[lo - b0:lo - b0 + n], out[lo:lo + n], w, buf, n, seq)
                        if on_chunk is not None:
                            on_chunk(lo, n)
                else:
                    cur = self._layer(cur, buf["ping"][:b] if li % 2 == 0 else buf["pong"][:b], w, buf, b, seq)
        return out

    def __call__(self, x_host, out_host=None):
        """Host entry: host tensor in, host tensor out (see forward_host)."""
        if out_host is None:
            out_host = torch.empty(tuple(x_host.shape), dtype=torch.float32, pin_memory=True)
        self.forward_host(x_host, out_host)
        torch.cuda.current_stream(self.device).synchronize()
        return out_host

    def host_chunks(self, bsz):
        """[(lo, n), ...]: the micro-batches forward_host moves and computes, in order."""
        mb = min(self.micro_batch, max(bsz, 1))
        if 64 <= bsz <= self.micro_batch:
            mb = (bsz + 1) // 2  # a batch that fits one micro-batch still moves in two, so that copies overlap compute
        # Only the first host->device and the last device->host copy are not hidden behind compute: a larger batch
        # starts and ends with a half-size micro-batch.
        edge = mb // 2 if bsz >= 2 * self.micro_batch and mb >= 64 else 0
        bounds, b0 = [], 0
        while b0 < bsz:
            if edge and b0 == 0:
                b = edge
            elif edge and bsz - b0 <= mb + edge and bsz - b0 > edge:
                b = bsz - b0 - edge
            else:
                b = min(mb, bsz - b0)
            bounds.append((b0, b))
            b0 += b
        return bounds

    def forward_host(self, x_host, out_host, out_device=None, on_chunk=None):
        """Host buffers in and out, copies overlapped with compute.

        The batch moves in micro-batches through three streams: host->device copies on a copy-in
        stream into two alternating staging buffers, the layers on the current stream, and
        device->host copies of finished micro-batches on a copy-out stream, ordered by events. With
        pinned host tensors the copies of micro-batch i+1 and i-1 run while micro-batch i computes.
        `out_device` ([B, S, hidden] on the device, optional) also keeps the result resident, e.g.
        for the output all-gather; `on_chunk(lo, n)` is called after the launches that complete samples
        [lo, lo+n) of it (the pieces are host_chunks(B)). Returns after enqueueing; the caller synchronises the current
        stream (the last device->host copy is joined into it).
        """
        if x_host.dim() != 3 or x_host.shape[2] != self.hidden or x_host.dtype != torch.float32:
            raise ValueError("expected a float32 [B, S, %d] host tensor" % self.hidden)
        if tuple(out_host.shape) != tuple(x_host.shape):
            raise ValueError("out_host must have the input's shape")
        bsz, seq, _ = x_host.shape
        bounds = self.host_chunks(bsz)
        mb = max(b for _, b in bounds)
        buf = self._buffers(mb, seq)
        if self._io is None or self._io[0] != (mb, seq):
            e = lambda: torch.empty(mb, seq, self.hidden, device=self.device, dtype=torch.float32)  # noqa: E731
            self._io = ((mb, seq), [e(), e()], [e(), e()], torch.cuda.Stream(self.device), torch.cuda.Stream(self.device))
        _, x_stage, y_stage, s_in, s_out = self._io
        main = torch.cuda.current_stream(self.device)
        s_in.wait_stream(main)   # staging buffers may still be in use by earlier work on the main stream
        s_out.wait_stream(main)
        ev_in, ev_done, ev_out = [], [], []
        for i, (b0, b) in enumerate(bounds):
            slot = i % 2
            with torch.cuda.stream(s_in):
                if i >= 2:
                    s_in.wait_event(ev_done[i - 2])  # the layers have consumed this staging buffer
                x_stage[slot][:b].copy_(x_host[b0:b0 + b], non_blocking=True)
                ev_in.append(s_in.record_event())
            main.wait_event(ev_in[i])
            if i >= 2:
                main.wait_event(ev_out[i - 2])  # the previous result in this slot has left for the host
            dst = out_device[b0:b0 + b] if out_device is not None else y_stage[slot][:b]
            cur = x_stage[slot][:b]
            for li, w in enumerate(self.layers):
                last = li + 1 == len(self.layers)
                nxt = dst if last else (buf["ping"][:b] if li % 2 == 0 else buf["pong"][:b])
                cur = self._layer(cur, nxt, w, buf, b, seq)
            ev_done.append(main.record_event())
            if on_chunk is not None:
                on_chunk(b0, b)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_done[i])
                out_host[b0:b0 + b].copy_(dst, non_blocking=True)
                ev_out.append(s_out.record_event())
        main.wait_stream(s_out)
        return out_host

    # -- work model (algorithmic figures used by the roofline report) ---------------------------------
    def flops_per_sequence(self, seq):
        h, f, nh, d = self.hidden, self.ffn, self.heads, self.head_dim
        per_layer = 2 * seq * (3 * h * h + h * h + 2 * f * h) + 4 * nh * seq * seq * d
        return per_layer * len(self.layers)
