"""Chain-fusion passes over an imported graph: the rewrites that turn the exported node chains into
the fused kernels of this library, in the style of the reference's subgraph replacements
(daceml/transformation/replacement.py:68-181, daceml/transformation/pad_conv_fusion.py:13-95).

    fuse_layernorm      ReduceMean-Sub-Pow-ReduceMean-Add-Sqrt-Div[-Mul-Add]   -> B200LayerNorm
    fuse_gelu           Div(sqrt 2)-Erf-Add(1)-Mul(x)-Mul(0.5)                 -> B200Gelu
    fuse_attention      Reshape/Transpose head split, MatMul-Mul|Div-Softmax-MatMul, head merge
                                                                               -> B200Attention
                        (+ the three projections that feed it, when they share their input
                                                                               -> B200SelfAttention)
    fold_transposes     Transpose (last two axes swapped) feeding MatMul's B   -> trans_b on the GEMM
    fuse_gemm_epilogues MatMul|Gemm - Add(bias) [- Relu | B200Gelu | Add(residual)], MatMul - Mul|Div(scalar)
                                                                               -> B200Gemm with an epilogue
    fuse_conv_relu      Conv(bias) - Relu                                      -> Conv with relu=1

Every pass only fires when all intermediate values of the pattern have no other consumer and are not
graph outputs, so the rewritten graph computes the same values as the node chain (up to the rounding
differences stated with each kernel). Host-only code.
"""
import math
from typing import List, Optional

import numpy as np

from .onnx_graph import GraphIR
from .onnx_wire import Node


class _View:
    """Producer / consumer maps of one graph state."""

    def __init__(self, ir: GraphIR):
        self.ir = ir
        self.prod = ir.producers()
        self.cons = ir.consumers()
        self.outs = set(ir.outputs)

    def only_consumer(self, name: str, op: Optional[str] = None) -> Optional[Node]:
        c = self.cons.get(name, [])
        if len(c) != 1 or name in self.outs:
            return None
        return c[0] if op is None or c[0].op_type == op else None

    def consumers_are(self, name: str, nodes: List[Node]) -> bool:
        c = self.cons.get(name, [])
        return name not in self.outs and len(c) == len(nodes) and {id(x) for x in c} == {id(x) for x in nodes}

    def scalar(self, name: str) -> Optional[float]:
        v = self.ir.consts.get(name)
        if v is None or v.size != 1:
            return None
        return float(v.reshape(-1)[0])

    def vector(self, name: str, length: int) -> bool:
        v = self.ir.consts.get(name)
        return v is not None and v.dtype == np.float32 and v.size == length and v.shape[-1:] == (length,)


def _other(node: Node, name: str) -> str:
    a, b = node.inputs[0], node.inputs[1]
    return b if a == name else a


def _last_axis(node: Node, rank: int) -> bool:
    axes = node.attr("axes")
    return axes is not None and len(axes) == 1 and axes[0] % rank == rank - 1 and node.attr("keepdims", 1) == 1


def fuse_layernorm(ir: GraphIR) -> int:
    count = 0
    while True:
        v = _View(ir)
        hit = None
        for m1 in ir.nodes:
            if m1.op_type != "ReduceMean":
                continue
            x = m1.inputs[0]
            rank = len(ir.shapes.get(x, ()))
            if rank == 0 or not _last_axis(m1, rank):
                continue
            sub = v.only_consumer(m1.outputs[0], "Sub")
            if sub is None or sub.inputs != [x, m1.outputs[0]]:
                continue
            c = v.cons.get(sub.outputs[0], [])
            pw = next((n for n in c if n.op_type == "Pow"), None)
            dv = next((n for n in c if n.op_type == "Div"), None)
            if pw is None or dv is None or not v.consumers_are(sub.outputs[0], [pw, dv]):
                continue
            if pw.inputs[0] != sub.outputs[0] or v.scalar(pw.inputs[1]) != 2.0:
                continue
            m2 = v.only_consumer(pw.outputs[0], "ReduceMean")
            if m2 is None or not _last_axis(m2, rank):
                continue
            ad = v.only_consumer(m2.outputs[0], "Add")
            if ad is None:
                continue
            eps = v.scalar(_other(ad, m2.outputs[0]))
            if eps is None or eps < 0:
                continue
            sq = v.only_consumer(ad.outputs[0], "Sqrt")
            if sq is None or v.only_consumer(sq.outputs[0]) is not dv or dv.inputs != [sub.outputs[0], sq.outputs[0]]:
                continue
            chain = [m1, sub, pw, m2, ad, sq, dv]
            final, gamma, beta = dv.outputs[0], "", ""
            length = ir.shapes[x][-1]
            ml = v.only_consumer(final, "Mul")
            if ml is not None and v.vector(_other(ml, final), length):
                gamma, final = _other(ml, final), ml.outputs[0]
                chain.append(ml)
                ab = v.only_consumer(final, "Add")
                if ab is not None and v.vector(_other(ab, final), length):
                    beta, final = _other(ab, final), ab.outputs[0]
                    chain.append(ab)
            hit = (chain, Node("B200LayerNorm", m1.name + "_ln", [x, gamma, beta], [final], {"epsilon": eps}))
            break
        if hit is None:
            return count
        ir.replace(*hit)
        count += 1


def fuse_gelu(ir: GraphIR) -> int:
    count = 0
    while True:
        v = _View(ir)
        hit = None
        for er in ir.nodes:
            if er.op_type != "Erf":
                continue
            dv = v.prod.get(er.inputs[0])
            if dv is None or dv.op_type != "Div" or v.only_consumer(dv.outputs[0]) is not er:
                continue
            c = v.scalar(dv.inputs[1])
            if c is None or abs(c - math.sqrt(2.0)) > 1e-6:
                continue
            x = dv.inputs[0]
            ad = v.only_consumer(er.outputs[0], "Add")
            if ad is None or v.scalar(_other(ad, er.outputs[0])) != 1.0:
                continue
            m1 = v.only_consumer(ad.outputs[0], "Mul")
            if m1 is None or _other(m1, ad.outputs[0]) != x:
                continue
            m2 = v.only_consumer(m1.outputs[0], "Mul")
            if m2 is None or v.scalar(_other(m2, m1.outputs[0])) != 0.5:
                continue
            hit = ([dv, er, ad, m1, m2], Node("B200Gelu", er.name + "_gelu", [x], [m2.outputs[0]], {}))
            break
        if hit is None:
            return count
        ir.replace(*hit)
        count += 1


def _head_split(v: _View, name: str, perm):
    """name = Transpose[perm](Reshape(src, [B, S, h, d])) with both single-consumer -> (src, [rs, tr], (B,S,h,d))."""
    tr = v.prod.get(name)
    if tr is None or tr.op_type != "Transpose" or list(tr.attr("perm") or []) != list(perm):
        return None
    if v.only_consumer(name) is None:
        return None
    rs = v.prod.get(tr.inputs[0])
    if rs is None or rs.op_type != "Reshape" or v.only_consumer(rs.outputs[0]) is not tr:
        return None
    src = rs.inputs[0]
    s_in, s4 = v.ir.shapes.get(src), v.ir.shapes.get(rs.outputs[0])
    if s_in is None or s4 is None or len(s_in) != 3 or len(s4) != 4:
        return None
    if s4[0] != s_in[0] or s4[1] != s_in[1] or s4[2] * s4[3] != s_in[2]:
        return None
    return src, [rs, tr], s4


def fuse_attention(ir: GraphIR) -> int:
    count = 0
    while True:
        v = _View(ir)
        hit = None
        for sm in ir.nodes:
            if sm.op_type != "Softmax":
                continue
            rank = len(ir.shapes[sm.inputs[0]])
            if rank != 4 or sm.attr("axis", 1) % rank != 3:
                continue
            sc = v.prod.get(sm.inputs[0])
            if sc is None or sc.op_type not in ("Mul", "Div") or v.only_consumer(sc.outputs[0]) is not sm:
                continue
            if sc.op_type == "Div":
                c = v.scalar(sc.inputs[1])
                scale = None if not c else 1.0 / c
                qk_name = sc.inputs[0]
            else:
                qk_name = sc.inputs[0] if v.scalar(sc.inputs[1]) is not None else sc.inputs[1]
                scale = v.scalar(_other(sc, qk_name))
            if scale is None or scale <= 0:
                continue
            qk = v.prod.get(qk_name)
            if qk is None or qk.op_type != "MatMul" or v.only_consumer(qk_name) is not sc:
                continue
            q = _head_split(v, qk.inputs[0], (0, 2, 1, 3))
            k = _head_split(v, qk.inputs[1], (0, 2, 3, 1))
            pv = v.only_consumer(sm.outputs[0], "MatMul")
            if q is None or k is None or pv is None or pv.inputs[0] != sm.outputs[0]:
                continue
            val = _head_split(v, pv.inputs[1], (0, 2, 1, 3))
            if val is None or not (q[2] == k[2] == val[2]):
                continue
            tr = v.only_consumer(pv.outputs[0], "Transpose")
            if tr is None or list(tr.attr("perm") or []) != [0, 2, 1, 3]:
                continue
            rs = v.only_consumer(tr.outputs[0], "Reshape")
            b, s, h, d = q[2]
            if rs is None or tuple(ir.shapes[rs.outputs[0]]) != (b, s, h * d):
                continue
            chain = q[1] + k[1] + val[1] + [qk, sc, sm, pv, tr, rs]
            hit = (chain, Node("B200Attention", sm.name + "_attention", [q[0], k[0], val[0]], [rs.outputs[0]],
                               {"heads": h, "scale": scale}))
            break
        if hit is None:
            break
        ir.replace(*hit)
        count += 1
    _merge_qkv(ir)
    return count


def _merge_qkv(ir: GraphIR):
    """B200Attention whose q, k, v are MatMul(x, W*) + bias* of one x: one projection GEMM instead of three."""
    while True:
        v = _View(ir)
        hit = None
        for at in ir.nodes:
            if at.op_type != "B200Attention":
                continue
            parts, chain, x = [], [], None
            for name in at.inputs:
                ad = v.prod.get(name)
                if ad is None or ad.op_type != "Add" or v.only_consumer(name) is not at:
                    break
                mm_out = next((i for i in ad.inputs if v.prod.get(i) is not None and v.prod[i].op_type == "MatMul"), None)
                if mm_out is None or v.only_consumer(mm_out) is not ad:
                    break
                mm, bias = v.prod[mm_out], _other(ad, mm_out)
                w = ir.consts.get(mm.inputs[1])
                if w is None or w.ndim != 2 or w.dtype != np.float32 or not v.vector(bias, w.shape[1]):
                    break
                if ir.consts[bias].ndim != 1 or (x is not None and mm.inputs[0] != x):
                    break
                x = mm.inputs[0]
                parts += [mm.inputs[1], bias]
                chain += [mm, ad]
            else:
                shapes = {ir.consts[parts[i]].shape for i in (0, 2, 4)}
                if len(shapes) == 1 and len(ir.shapes[x]) == 3:
                    hit = (chain + [at], Node("B200SelfAttention", at.name, [x] + parts, list(at.outputs),
                                              dict(at.attrs)))
                    break
        if hit is None:
            return
        ir.replace(*hit)


def fold_transposes(ir: GraphIR) -> int:
    """MatMul(A, Transpose(B)) where the transpose swaps the last two axes (possibly after another
    permutation): the swap becomes the GEMM's trans_b flag; an identity remainder disappears."""
    count = 0
    while True:
        v = _View(ir)
        hit = None
        for mm in ir.nodes:
            if mm.op_type != "MatMul" or mm.attr("trans_b", 0):
                continue
            tr = v.prod.get(mm.inputs[1])
            if tr is None or tr.op_type != "Transpose" or v.only_consumer(tr.outputs[0]) is not mm:
                continue
            rank = len(ir.shapes[tr.inputs[0]])
            perm = list(tr.attr("perm") or list(range(rank))[::-1])
            if rank < 2:
                continue
            rest = perm[:-2] + [perm[-1], perm[-2]]  # perm = rest followed by a swap of the last two axes
            hit = (mm, tr, rest)
            break
        if hit is None:
            return count
        mm, tr, rest = hit
        mm.attrs["trans_b"] = 1
        if rest == list(range(len(rest))):
            mm.inputs[1] = tr.inputs[0]
            ir.nodes = [n for n in ir.nodes if n is not tr]
        else:
            tr.attrs["perm"] = rest
            src = ir.shapes[tr.inputs[0]]
            ir.shapes[tr.outputs[0]] = tuple(src[p] for p in rest)
        count += 1


def fuse_gemm_epilogues(ir: GraphIR) -> int:
    count = 0
    while True:
        v = _View(ir)
        hit = None
        for mm in ir.nodes:
            if mm.op_type == "MatMul":
                y = mm.outputs[0]
                n_out = ir.shapes[y][-1]
                trans_b = int(mm.attr("trans_b", 0))
                nxt = v.only_consumer(y)
                if nxt is not None and nxt.op_type in ("Mul", "Div") and v.scalar(_other(nxt, y)) is not None and \
                        (nxt.op_type == "Mul" or nxt.inputs[0] == y):
                    c = v.scalar(_other(nxt, y))
                    if nxt.op_type == "Div" and c == 0.0:
                        continue
                    # Mul by c, or Div by a power of two (exact as a multiplication by the reciprocal)
                    if nxt.op_type == "Div" and math.frexp(c)[0] != 0.5:
                        continue
                    scale = c if nxt.op_type == "Mul" else 1.0 / c
                    hit = ([mm, nxt], Node("B200Gemm", mm.name, [mm.inputs[0], mm.inputs[1], "", ""], [nxt.outputs[0]],
                                           {"trans_b": trans_b, "epilogue": "scale", "scale": scale}))
                    break
                if nxt is None or nxt.op_type != "Add":
                    continue
                bias = _other(nxt, y)
                if not (v.vector(bias, n_out) and ir.consts[bias].ndim == 1):
                    continue
                a_in, b_in = mm.inputs[0], mm.inputs[1]
            elif mm.op_type == "Gemm":
                if mm.attr("alpha", 1.0) != 1.0 or mm.attr("beta", 1.0) != 1.0 or mm.attr("transA", 0):
                    continue
                if len(mm.inputs) < 3 or not mm.inputs[2]:
                    continue
                y = mm.outputs[0]
                n_out = ir.shapes[y][-1]
                bias = mm.inputs[2]
                if not (v.vector(bias, n_out) and ir.consts[bias].ndim == 1):
                    continue
                trans_b = int(mm.attr("transB", 0))
                a_in, b_in = mm.inputs[0], mm.inputs[1]
                nxt = mm
            else:
                continue
            chain = [mm] if nxt is mm else [mm, nxt]
            out, epi, residual = nxt.outputs[0], "bias", ""
            act = v.only_consumer(out)
            if act is not None and act.op_type == "Relu":
                chain.append(act)
                out, epi = act.outputs[0], "bias_relu"
            elif act is not None and act.op_type == "B200Gelu":
                chain.append(act)
                out, epi = act.outputs[0], "bias_gelu"
            elif act is not None and act.op_type == "Add":
                other = _other(act, out)
                if other not in ir.consts and ir.shapes.get(other) == ir.shapes[out] and other != out:
                    chain.append(act)
                    out, epi, residual = act.outputs[0], "bias_residual", other
            hit = (chain, Node("B200Gemm", mm.name, [a_in, b_in, bias, residual], [out],
                               {"trans_b": trans_b, "epilogue": epi, "scale": 1.0}))
            break
        if hit is None:
            return count
        ir.replace(*hit)
        count += 1


def fuse_conv_relu(ir: GraphIR) -> int:
    count = 0
    v = _View(ir)
    for cv in list(ir.nodes):
        if cv.op_type != "Conv" or len(cv.inputs) < 3 or not cv.inputs[2] or cv.attr("relu", 0):
            continue
        act = v.only_consumer(cv.outputs[0], "Relu")
        if act is None:
            continue
        cv.attrs["relu"] = 1
        cv.outputs[0] = act.outputs[0]
        ir.nodes = [n for n in ir.nodes if n is not act]
        v = _View(ir)
        count += 1
    return count


def run_all(ir: GraphIR) -> dict:
    """Apply every pass in dependency order; returns how often each fired."""
    stats = {"layernorm": fuse_layernorm(ir), "gelu": fuse_gelu(ir), "attention": fuse_attention(ir),
             "transposes": fold_transposes(ir), "gemm_epilogues": fuse_gemm_epilogues(ir),
             "conv_relu": fuse_conv_relu(ir)}
    return stats
