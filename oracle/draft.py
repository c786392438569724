"""CPU restatement of the reference's DFlash 2 drafter (Sources/SploshRuntime/DraftModel.swift, Sources/Shaders/draft.metal)
in numpy. TEST INFRASTRUCTURE ONLY: only tests/ may import this.

Parity unpinned: the reference holds no test, golden vector or fixture for its drafter, and its code cannot run here
(Swift + Metal). The linear products go through the oracle's q4 GEMM (oracle.gemm_q4, pinned on the reference's vectors);
everything else below follows the cited lines.
"""
import numpy as np

from . import oracle as O

HEAD_DIM = 128
F = np.float32


def bf16_bits(x):
    """DraftModel.bf16 (:721-724): fp32 -> bf16 bits, nearest even."""
    bits = np.ascontiguousarray(x, F).view(np.uint32).astype(np.uint64)
    return ((bits + 0x7FFF + ((bits >> 16) & 1)) >> 16).astype(np.uint16)


def bits_float(bits):
    return (np.asarray(bits, np.uint16).astype(np.uint32) << 16).view(F)


def _rounded(x):
    """Swift's rounded(): nearest, ties away from zero (arguments here are finite)."""
    t = np.trunc(x)
    return (t + np.where(np.abs(x - t) >= F(0.5), np.sign(x), F(0))).astype(F)


def _codes(values, bias, scale):
    return np.minimum(F(15), np.maximum(F(0), _rounded((values - bias) / scale))).astype(F)


def _seq_sum(terms):
    """Sum over the last axis in index order, in fp32 (the reference's loops)."""
    acc = np.zeros(terms.shape[:-1], F)
    for i in range(terms.shape[-1]):
        acc = (acc + terms[..., i]).astype(F)
    return acc


def _error(x, scale_bits, bias_bits):
    scale, bias = bits_float(scale_bits)[:, None], bits_float(bias_bits)[:, None]
    with np.errstate(all="ignore"):
        code = _codes(x, bias, scale)
        difference = (x - (bias + scale * code).astype(F)).astype(F)
        total = _seq_sum((difference * difference).astype(F))
    bad = ~((scale[:, 0] > 0) & np.isfinite(scale[:, 0]) & np.isfinite(bias[:, 0]))
    return np.where(bad, F(np.inf), total).astype(F)


def quantize(source_bits, fitted=True):
    """DraftModel.quantize + fitRange (:635-719) on bf16 bits [rows][inner], row-major: (packed, scale bits, bias bits)."""
    src = np.ascontiguousarray(source_bits, np.uint16)
    rows, inner = src.shape
    groups = inner // 64
    x = bits_float(src).reshape(rows * groups, 64)
    lowest, highest = x.min(axis=1), x.max(axis=1)
    spread = highest > lowest
    with np.errstate(all="ignore"):
        scale_bits = bf16_bits(np.where(spread, ((highest - lowest).astype(F) / F(15)).astype(F), F(1)))
    bias_bits = bf16_bits(lowest)
    if fitted:
        best_s, best_b = scale_bits.copy(), bias_bits.copy()
        best_error = _error(x, best_s, best_b)
        rng_ = (highest - lowest).astype(F)
        count = F(64)
        for low in (F(0), F(0.04), F(0.08)):
            for high in (F(0), F(0.04), F(0.08)):
                with np.errstate(all="ignore"):
                    scale = ((rng_ * ((F(1) - low).astype(F) - high).astype(F)).astype(F) / F(15)).astype(F)
                    bias = (lowest + (low * rng_).astype(F)).astype(F)
                    live = spread.copy()
                    for _ in range(2):
                        code = _codes(x, bias[:, None], scale[:, None])
                        sum_code, sum_value = _seq_sum(code), _seq_sum(x)
                        sum_code2, sum_code_value = _seq_sum((code * code).astype(F)), _seq_sum((code * x).astype(F))
                        determinant = ((count * sum_code2).astype(F) - (sum_code * sum_code).astype(F)).astype(F)
                        live = live & (determinant > 0)
                        refitted = (((count * sum_code_value).astype(F) - (sum_code * sum_value).astype(F)).astype(F) / determinant).astype(F)
                        live = live & (refitted > 0)
                        scale = np.where(live, refitted, scale).astype(F)
                        bias = np.where(live, ((sum_value - (refitted * sum_code).astype(F)).astype(F) / count).astype(F), bias).astype(F)
                    cs, cb = bf16_bits(scale), bf16_bits(bias)
                    candidate_error = _error(x, cs, cb)
                better = spread & (candidate_error < best_error)
                best_s = np.where(better, cs, best_s); best_b = np.where(better, cb, best_b)
                best_error = np.where(better, candidate_error, best_error)
        scale_bits, bias_bits = best_s, best_b
    scale, bias = bits_float(scale_bits)[:, None], bits_float(bias_bits)[:, None]
    with np.errstate(all="ignore"):
        codes = _codes(x, bias, scale).astype(np.uint32).reshape(rows * groups, 8, 8)
    words = np.zeros((rows * groups, 8), np.uint32)
    for nibble in range(8):
        words |= codes[:, :, nibble] << np.uint32(4 * nibble)
    return words.reshape(rows, inner // 8), scale_bits.reshape(rows, groups), bias_bits.reshape(rows, groups)


def rope(x, paired, i, position, theta):
    """spd_rope (draft.metal:13-19): element i of a 128-wide head at `position`, pairs (i, i + 64)."""
    half = HEAD_DIM // 2
    slot = np.where(i < half, i, i - half).astype(np.float64)
    angle = np.float64(position) * np.power(np.float64(theta), -(2.0 * slot) / HEAD_DIM)
    return x * np.cos(angle) + np.where(i < half, -paired, paired) * np.sin(angle)


def select(ids, values, hidden_rows, hidden_projection, predecessor, successor, anchor, temperature=0.0, random_state=0):
    """CandidateSelector.select (DraftModel.swift:479-531) for one request, in float64. Returns tokens, probabilities, state, and
    the margin between the two best scores of every position (a near-tie may fall either way in fp32)."""
    ids = np.asarray(ids); values = np.asarray(values, np.float64)
    drafted, k = ids.shape
    proj = np.asarray(hidden_projection, np.float64)
    tokens, probabilities, margins = [], [], []
    before_token = anchor
    state = int(random_state)
    for position in range(drafted):
        projected = proj @ np.asarray(hidden_rows[position], np.float64)
        gated = bits_float(predecessor[before_token]).astype(np.float64) * projected
        scores = values[position] + bits_float(successor[ids[position]]).astype(np.float64) @ gated
        order = np.sort(scores)
        margins.append(order[-1] - order[-2] if k > 1 else np.inf)
        if temperature > 0:
            q = np.exp((scores - scores.max()) / temperature)
            q /= q.sum()
            state = (state + 0x9E3779B97F4A7C15) & 0xFFFFFFFFFFFFFFFF
            z = state
            z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & 0xFFFFFFFFFFFFFFFF
            z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & 0xFFFFFFFFFFFFFFFF
            z ^= z >> 31
            draw = float(np.float32(z >> 40) / np.float32(1 << 24))
            choice = k - 1
            for index in range(k):
                draw -= q[index]
                if draw <= 0:
                    choice = index
                    break
            probabilities.append(q)
        else:
            choice = int(np.argmax(scores))        # the first of equal scores, as the reference's strict comparison keeps it
        before_token = int(ids[position][choice])
        tokens.append(before_token)
    return tokens, (np.array(probabilities) if temperature > 0 else None), state, np.array(margins)


class Draft:
    """The drafter over a target `oracle.Model` (its embedding and head) with the checkpoint's tensors as bf16 bits by name."""

    def __init__(self, model, config, tensors, taps):
        self.model, self.c, self.g = model, config, model.g
        self.hidden, self.inter, self.vocab = self.g.hidden, self.g.inter, self.g.vocab
        self.groups = self.hidden // config.group_size
        self.kv = config.kv_heads * HEAD_DIM
        self.attention = config.heads * HEAD_DIM
        self.t = tensors
        self.q4 = {}
        for name, bits in tensors.items():
            if name.endswith("proj.weight") or name.endswith("projection.weight") and "kernel_projection" in name or name == "fc.weight":
                self.q4[name] = quantize(bits, fitted=not config.minmax_ranges)
        slots = 8
        self.k_ring = np.zeros((config.layers, slots, config.ring_capacity, config.kv_heads, HEAD_DIM), np.float16)
        self.v_ring = np.zeros_like(self.k_ring)
        self.first, self.end = [0] * slots, [0] * slots
        self.taps = taps

    def linear(self, name, x):
        return O.gemm_q4(*self.q4[name], x)

    def norm(self, x, name):
        x = np.asarray(x, F)
        inv = 1.0 / np.sqrt((x.astype(np.float64) ** 2).mean(axis=1, keepdims=True) + self.g.eps)
        return (x * inv * bits_float(self.t[name])).astype(F)

    def store(self, layer, k, v, slots, positions):
        """sp_draft_kv_store (draft.metal:59-100)."""
        c = self.c
        w = bits_float(self.t[f"layers.{layer}.self_attn.k_norm.weight"]).astype(np.float64)
        i = np.arange(HEAD_DIM)
        pi = np.where(i < HEAD_DIM // 2, i + HEAD_DIM // 2, i - HEAD_DIM // 2)
        for r in range(len(slots)):
            kk = np.asarray(k[r], np.float64).reshape(c.kv_heads, HEAD_DIM)
            inv = 1.0 / np.sqrt((kk ** 2).mean(axis=1, keepdims=True) + self.g.eps)
            x = kk * inv * w
            self.k_ring[layer, slots[r], positions[r] % c.ring_capacity] = rope(x, x[:, pi], i, positions[r], self.g.rope_theta).astype(np.float16)
            self.v_ring[layer, slots[r], positions[r] % c.ring_capacity] = np.asarray(v[r], F).reshape(c.kv_heads, HEAD_DIM).astype(np.float16)

    def push_context(self, features, slots, positions):
        """DraftModel.pushContext (:328-359) on the target's feature rows [n][taps x hidden]."""
        for slot, position in zip(slots, positions):
            if position != self.end[slot]:
                self.first[slot] = position
            self.end[slot] = position + 1
        hidden = self.linear("fc.weight", np.asarray(features, F))
        normed = self.norm(hidden, "hidden_norm.weight")
        for layer in range(self.c.layers):
            k = self.linear(f"layers.{layer}.self_attn.k_proj.weight", normed)
            v = self.linear(f"layers.{layer}.self_attn.v_proj.weight", normed)
            self.store(layer, k, v, slots, positions)

    def conv(self, x, dyn, base_name, which, offsets):
        """sp_dyn_conv (draft.metal:21-57)."""
        base = bits_float(self.t[base_name]).reshape(4, self.hidden)
        rows = x.shape[0]
        group = np.arange(self.hidden) // self.c.group_size
        out = np.zeros((rows, self.hidden), F)
        dyn = np.asarray(dyn, F).reshape(rows, 4, self.groups)
        for t in range(rows):
            acc = np.zeros(self.hidden, F)
            for o in range(2):
                if offsets[t] < o:
                    continue
                tap = which * 2 + o
                acc = acc + (base[tap] + dyn[t, tap][group]) * x[t - o]
            out[t] = acc
        return out

    def attend(self, layer, q, slots, positions, lo, hi):
        """sp_draft_attention (draft.metal:102-192), in float64."""
        c = self.c
        w = bits_float(self.t[f"layers.{layer}.self_attn.q_norm.weight"]).astype(np.float64)
        i = np.arange(HEAD_DIM)
        pi = np.where(i < HEAD_DIM // 2, i + HEAD_DIM // 2, i - HEAD_DIM // 2)
        rows = q.shape[0]
        out = np.zeros((rows, c.heads, HEAD_DIM), F)
        per = c.heads // c.kv_heads
        for r in range(rows):
            qq = np.asarray(q[r], np.float64).reshape(c.heads, HEAD_DIM)
            inv = 1.0 / np.sqrt((qq ** 2).mean(axis=1, keepdims=True) + self.g.eps)
            x = qq * inv * w
            query = rope(x, x[:, pi], i, positions[r], self.g.rope_theta)
            first_visible = positions[r] + 1 - c.window if positions[r] + 1 > c.window else 0
            span = np.arange(max(lo[r], first_visible), hi[r])
            ring = span % c.ring_capacity
            for head in range(c.heads):
                kvh = head // per
                keys = self.k_ring[layer, slots[r], ring, kvh].astype(np.float64)
                values = self.v_ring[layer, slots[r], ring, kvh].astype(np.float64)
                scores = keys @ query[head] / np.sqrt(HEAD_DIM)
                p = np.exp(scores - scores.max())
                out[r, head] = (p @ values / p.sum()).astype(F)
        return out.reshape(rows, c.heads * HEAD_DIM)

    def propose(self, requests, temperature=0.0, vocab_limit=None, random_state=0):
        """DraftModel.propose (:380-477): proposals, plus the logits and selected hidden rows they came from."""
        c = self.c
        tokens, slots, positions, lo, hi, offsets, gather, first_picked = [], [], [], [], [], [], [], []
        for r in requests:
            first = self.first[r.slot] if self.end[r.slot] == r.start else r.start
            first_picked.append(len(gather))
            for offset in range(r.block):
                if offset > 0:
                    gather.append(len(tokens))
                tokens.append(r.anchor if offset == 0 else c.mask_token)
                slots.append(r.slot); positions.append(r.start + offset); lo.append(first)
                hi.append(r.start + (c.block_size if r.isolate_prefix and offset < c.block_size else r.block))
                offsets.append(offset)
        packed, scales, biases = self.model.q4(-1, "embed")
        tok = np.array(tokens)
        dh = O.dequant_mlx4(packed[tok], bits_float(scales[tok]), bits_float(biases[tok]), self.hidden)
        for layer in range(c.layers):
            p = f"layers.{layer}."
            x = self.norm(dh, p + "input_layernorm.weight")
            dyn = self.linear(p + "attention_conv.kernel_projection.weight", x)
            xc = self.conv(x, dyn, p + "attention_conv.base_kernel", 0, offsets)
            q, k, v = (self.linear(p + f"self_attn.{n}_proj.weight", xc) for n in "qkv")
            self.store(layer, k, v, slots, positions)
            ao = self.attend(layer, q, slots, positions, lo, hi)
            t = self.linear(p + "self_attn.o_proj.weight", ao)
            dh = (dh + self.conv(t, dyn, p + "attention_conv.base_kernel", 1, offsets)).astype(F)
            t_attn, dh_attn, dyn_attn = t, dh, dyn
            x = self.norm(dh, p + "post_attention_layernorm.weight")
            dyn = self.linear(p + "mlp_conv.kernel_projection.weight", x)
            xc = self.conv(x, dyn, p + "mlp_conv.base_kernel", 0, offsets)
            gate, up = self.linear(p + "mlp.gate_proj.weight", xc), self.linear(p + "mlp.up_proj.weight", xc)
            act = O.bf16_round((gate / (1.0 + np.exp(-gate.astype(np.float64))) * up).astype(F))
            t = self.linear(p + "mlp.down_proj.weight", act)
            dh = (dh + self.conv(t, dyn, p + "mlp_conv.base_kernel", 1, offsets)).astype(F)
            trace = dict(x=x, xc=xc, dyn=dyn, q=q, ao=ao, t=t, gate=act, t_attn=t_attn, dh_attn=dh_attn, dyn_attn=dyn_attn)
        dn = self.norm(dh, "norm.weight")
        selected = dn[np.array(gather)]
        logits = O.gemm_q4(*self.model.q4(-1, "head"), selected)
        return dict(logits=logits, selected=selected, first_picked=first_picked, residual=dh, trace=trace)
