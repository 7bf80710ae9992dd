"""One decoder layer of the CPU oracle, step by step, with its intermediate activations.

TEST INFRASTRUCTURE.  oracle.binding.Model.forward returns only the layer's output; the strict layer
parity test needs the activations at the points where the forward pass re-quantises them (attention
output, residual after the attention block, SwiGLU output), so the same arithmetic is assembled here
from the oracle's primitives in the order orc_model_forward applies them (oracle/kquant_oracle.c,
"whole stage").  tests/test_layer_oracle_cpu.py checks that this assembly reproduces Model.forward
bit for bit on dense models (and to f32 rounding of the router's dot products on expert models).

Why the segments exist: a Q8 activation code is rint(x / d).  Two correct implementations whose
inputs to a quantiser differ in the last bits of an f32 sum (another order of accumulation, an
online softmax against a two-pass one, an f16 cache element rounded the other way) occasionally get
neighbouring codes for one element.  One such code changes the quantiser's output by d, not by the
1e-7 the inputs differed by, and the next quantiser amplifies it again: a small perturbation delta
becomes about sqrt(delta * d).  Measured on a 3B-shape layer: one flipped code at the attention
output moves that row of the layer output by 9e-3 of max |ref|.  So the layer is compared segment by
segment, each segment starting at a quantiser whose input both sides share exactly (the quantiser is
bit-reproducible, RMSNorm carries its sum of squares in double on both sides), and inside a segment
the hot-path bound of 1e-3 holds without exception.
"""
import numpy as np

from oracle import binding as orc


class LayerOracle:
    """blk.<l> of an oracle.binding.Model; KV cache for one sequence held here (f16 bits)"""

    def __init__(self, model, cfg, layer):
        self.m, self.c, self.l = model, dict(cfg), layer
        c = self.c
        self.h, self.nh, self.nkv, self.hd = c["n_embd"], c["n_head"], c["n_head_kv"], c["head_dim"]
        self.eps, self.theta, self.neox = c.get("rms_eps", 1e-6), c.get("rope_theta", 1e6), c.get("rope_neox", 1)
        self.n_expert = c.get("n_expert", 0)
        self.kc = np.zeros((c["n_ctx"], self.nkv, self.hd), np.uint16)
        self.vc = np.zeros((c["n_ctx"], self.nkv, self.hd), np.uint16)

    # ---- tensors
    def _t(self, what):
        return self.m.tensor(f"blk.{self.l}.{what}")

    def _f32(self, what):
        return self._t(what)[1].view(np.float32)

    def _has(self, what):
        try:
            self._t(what)
            return True
        except KeyError:
            return False

    def _mm(self, what, a, N, K):
        ty, data, _ = self._t(what)
        return orc.mul_mat(ty, data, a, N, K)

    # ---- segments
    def attention_block(self, x, pos0):
        """x [T, h] -> attention output [T, n_head * hd] (writes the KV cache rows pos0 .. pos0 + T)"""
        T = x.shape[0]
        h, nh, nkv, hd = self.h, self.nh, self.nkv, self.hd
        xn = orc.rms_norm(x, self._f32("attn_norm.weight"), self.eps)
        q = self._mm("attn_q.weight", xn, nh * hd, h)
        k = self._mm("attn_k.weight", xn, nkv * hd, h)
        v = self._mm("attn_v.weight", xn, nkv * hd, h)
        if self._has("attn_q.bias"):
            q = q + self._f32("attn_q.bias")
            k = k + self._f32("attn_k.bias")
            v = v + self._f32("attn_v.bias")
        if self._has("attn_q_norm.weight"):
            q = orc.rms_norm(q.reshape(T * nh, hd), self._f32("attn_q_norm.weight"), self.eps).reshape(T, nh * hd)
            k = orc.rms_norm(k.reshape(T * nkv, hd), self._f32("attn_k_norm.weight"), self.eps).reshape(T, nkv * hd)
        pos = np.arange(pos0, pos0 + T, dtype=np.int32)
        qr = orc.rope(q.reshape(T, nh, hd), pos, self.theta, self.neox)
        kr = orc.rope(k.reshape(T, nkv, hd), pos, self.theta, self.neox)
        self.kc[pos0:pos0 + T] = orc.f32_to_f16(kr)
        self.vc[pos0:pos0 + T] = orc.f32_to_f16(v.reshape(T, nkv, hd))
        return orc.attention(qr, self.kc, self.vc, pos0).reshape(T, nh * hd)

    def attention_output(self, x, att):
        """x1 = x + Wo . att"""
        return x + self._mm("attn_output.weight", att, self.h, self.nh * self.hd)

    def ffn_activation(self, x1):
        """dense: SwiGLU output g [T, n_ff]"""
        ff = self.c["n_ff"]
        xn = orc.rms_norm(x1, self._f32("ffn_norm.weight"), self.eps)
        return orc.swiglu(self._mm("ffn_gate.weight", xn, ff, self.h), self._mm("ffn_up.weight", xn, ff, self.h))

    def ffn_output(self, x1, g):
        """dense: out = x1 + Wdown . g"""
        return x1 + self._mm("ffn_down.weight", g, self.h, self.c["n_ff"])

    def moe_block(self, x1, mask=None):
        """expert layer: out = x1 + sum_s w_s * down_e(swiglu(gate_e xn, up_e xn))"""
        h, E, ku, fe = self.h, self.n_expert, self.c["n_expert_used"], self.c["n_ff_exp"]
        T = x1.shape[0]
        xn = orc.rms_norm(x1, self._f32("ffn_norm.weight"), self.eps)
        wr = self._f32("ffn_gate_inp.weight").reshape(E, h)
        logits = np.empty((T, E), np.float32)
        for t in range(T):  # f32 dot products, element by element as the oracle's loop does
            logits[t] = (wr * xn[t]).astype(np.float32).cumsum(-1, dtype=np.float32)[:, -1]
        ids, w = orc.moe_route(logits, ku, mask)
        gty, gd, _ = self._t("ffn_gate_exps.weight")
        uty, ud, _ = self._t("ffn_up_exps.weight")
        dty, dd, _ = self._t("ffn_down_exps.weight")
        gd, ud, dd = gd.reshape(E, -1), ud.reshape(E, -1), dd.reshape(E, -1)
        out = np.empty_like(x1)
        for t in range(T):
            acc = np.zeros(h, np.float32)
            for s in range(ku):
                e = ids[t, s]
                g = orc.swiglu(orc.mul_mat(gty, gd[e], xn[t:t + 1], fe, h), orc.mul_mat(uty, ud[e], xn[t:t + 1], fe, h))
                acc = acc + w[t, s] * orc.mul_mat(dty, dd[e], g, h, fe)[0]
            out[t] = x1[t] + acc
        return out

    def forward(self, x, pos0):
        """-> dict of the layer's activations"""
        att = self.attention_block(x, pos0)
        x1 = self.attention_output(x, att)
        if self.n_expert > 0:
            return dict(att=att, x1=x1, out=self.moe_block(x1))
        g = self.ffn_activation(x1)
        return dict(att=att, x1=x1, g=g, out=self.ffn_output(x1, g))
