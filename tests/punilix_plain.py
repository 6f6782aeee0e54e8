"""Plain, slow restatement of the Punilix design in float64 torch, one function per mechanism.

Independent of the product path: it reads no product code and is only used by tests as the oracle.
Notation: x is the residual stream [T, W]; every linear weight is [out, in] and applied as x @ W.T.

  layer:        h = group_rms(x);  x <- x + mixer(h) + ff(h)          (one norm, both sublayers read it)
  group_rms:    the vector is cut into `groups` equal parts, each part p -> p / sqrt(mean(p^2) + eps), whole times w
  general_delta per head, S in R^{dim x dim} (key channel x value channel), S_0 = 0:
                  d = exp(-e^{-1/2} * sigmoid(W_w2 tanh(W_w1 h) + w0))      (decay per key channel)
                  a = sigmoid(W_a h + b_a)                                  (removal rate per key channel)
                  u = k / sqrt(sum(k^2) + 1e-6)
                  S_t = diag(d) S_{t-1} - (a*u) (u^T S_{t-1}) + k v^T ;  o_t = S_t^T r
                o / rms(o) per head, times weight, times sigmoid(W_g h), then W_o
  latent_attention: queries through a normed latent, keys / values from a normed shared latent c plus one rotated key part
                shared by all heads; interleaved rotary pairs with YaRN-blended frequencies; causal softmax; sigmoid output gate
  ff:           g = min(W_gate h, L); u = clamp(W_up h, -L, L); y = g * sigmoid(1.702 g) * (u + 1); W_down y
  table moe:    a [vocab, top] integer table names each token id's experts, each weighted 1/top
  output:       group_rms with the final weight, head, then cap * tanh(logits / cap)
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def group_rms(x, w, groups, eps):
    T, W = x.shape
    p = x.reshape(T, groups, W // groups)
    p = p / torch.sqrt((p * p).mean(-1, keepdim=True) + eps)
    return p.reshape(T, W) * w


def plain_rms(x, w, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


def clamped_glu(h, wg, wu, wd, limit):
    g = torch.clamp(h @ wg.T, max=limit)
    u = torch.clamp(h @ wu.T, -limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ wd.T


def table_moe(h, tokens, table, experts, limit):
    """experts: list of (gate, up, down); table [vocab, top] integer."""
    out = torch.zeros(h.shape[0], experts[0][2].shape[0], dtype=h.dtype)
    top = table.shape[1]
    for t, tok in enumerate(tokens):
        for e in table[tok].tolist():
            wg, wu, wd = experts[e]
            out[t] += clamped_glu(h[t:t + 1], wg, wu, wd, limit)[0] / top
    return out


def general_delta(h, p, heads, dim, eps, state):
    """p: dict of the mixer's tensors; state: [heads, dim, dim] carried across calls (updated in place)."""
    T = h.shape[0]
    r = (h @ p["r"].T).reshape(T, heads, dim)
    k = (h @ p["k"].T).reshape(T, heads, dim)
    v = (h @ p["v"].T).reshape(T, heads, dim)
    d = torch.exp(-math.exp(-0.5) * torch.sigmoid(torch.tanh(h @ p["w1"].T) @ p["w2"].T + p["w0"])).reshape(T, heads, dim)
    a = torch.sigmoid(h @ p["a"].T + p["a.b"]).reshape(T, heads, dim)
    u = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    o = torch.zeros(T, heads, dim, dtype=h.dtype)
    for t in range(T):
        for n in range(heads):
            S = state[n]
            z = u[t, n] @ S                                   # u^T S_{t-1}
            S = d[t, n][:, None] * S - (a[t, n] * u[t, n])[:, None] * z[None, :] + k[t, n][:, None] * v[t, n][None, :]
            state[n] = S
            o[t, n] = S.T @ r[t, n]
    o = o / torch.sqrt((o * o).mean(-1, keepdim=True) + eps)
    o = o.reshape(T, heads * dim) * p["norm"] * torch.sigmoid(h @ p["g"].T)
    return o @ p["o"].T


def rotary_frequencies(rot):
    dims, base = rot["dims"], rot["base"]
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=F64)
    sc = rot.get("scaling")
    mult = 1.0
    if sc:
        def where(t):
            return dims * math.log(sc["original"] / (2 * math.pi * t)) / (2 * math.log(base))
        lo = max(math.floor(where(sc["fast"])), 0)
        hi = min(math.ceil(where(sc["slow"])), dims - 1)
        ramp = torch.tensor([min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0) for i in range(dims // 2)], dtype=F64)
        f = f / sc["factor"] * ramp + f * (1 - ramp)
        mult = 0.1 * math.log(sc["factor"]) + 1.0
    return f, mult


def rotate_pairs(x, positions, rot):
    """x [T, ..., n]: the first rot['dims'] entries are rotated as interleaved pairs (2i, 2i+1), the rest pass."""
    f, mult = rotary_frequencies(rot)
    dims = rot["dims"]
    # the angle is formed in 32-bit, like the product does
    ang = (positions.to(torch.float32)[:, None] * f.to(torch.float32)[None, :]).to(F64)
    cos, sin = torch.cos(ang) * mult, torch.sin(ang) * mult
    while cos.dim() < x.dim():
        cos, sin = cos.unsqueeze(1), sin.unsqueeze(1)
    a, b = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = a * cos - b * sin
    out[..., 1:dims:2] = b * cos + a * sin
    return out


def latent_attention(h, p, m, eps, positions, cache):
    """m: the mixer's sizes; cache: dict with 'c' [n, kv_rank] and 'kr' [n, rot_dim] of earlier tokens (extended in place)."""
    T = h.shape[0]
    H, dn, dr, dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    cq = plain_rms(h @ p["dq"].T, p["dq.norm"], eps)
    q = (cq @ p["uq"].T).reshape(T, H, dn + dr)
    q_n, q_r = q[..., :dn], rotate_pairs(q[..., dn:], positions, m["rot"])
    kv = h @ p["dkv"].T
    c = plain_rms(kv[:, :R], p["dkv.norm"], eps)
    kr = rotate_pairs(kv[:, R:], positions, m["rot"])
    cache["c"] = torch.cat([cache["c"], c])
    cache["kr"] = torch.cat([cache["kr"], kr])
    C, KR = cache["c"], cache["kr"]
    n = C.shape[0]
    k_n = (C @ p["uk"].T).reshape(n, H, dn)
    val = (C @ p["uv"].T).reshape(n, H, dv)
    s = (torch.einsum("thd,nhd->htn", q_n, k_n) + torch.einsum("thd,nd->htn", q_r, KR)) * m["scale"]
    key_pos = torch.arange(n)
    mask = key_pos[None, :] <= positions[:, None]
    s = s.masked_fill(~mask[None], float("-inf"))
    w = torch.softmax(s, -1)
    o = torch.einsum("htn,nhd->thd", w, val).reshape(T, H * dv)
    o = o * torch.sigmoid(h @ p["g"].T)
    return o @ p["o"].T


class PlainModel:
    """Holds float64 copies of the tensors and the per-sequence state; `step(tokens)` feeds the next tokens of one sequence."""

    def __init__(self, config, tensors):
        self.cfg = config
        self.t = {k: (v.to(F64) if v.is_floating_point() else v) for k, v in tensors.items()}
        self.reset()

    def reset(self):
        self.pos = 0
        self.state = []
        for L in self.cfg["layers"]:
            mx = L["mixer"]
            if L["type"] == "general_delta":
                self.state.append(torch.zeros(mx["heads"], mx["dim"], mx["dim"], dtype=F64))
            else:
                self.state.append({"c": torch.zeros(0, mx["kv_rank"], dtype=F64), "kr": torch.zeros(0, mx["rot_dim"], dtype=F64)})

    def sub(self, prefix):
        n = len(prefix)
        return {k[n:]: v for k, v in self.t.items() if k.startswith(prefix)}

    def step(self, tokens, layer_outputs=None):
        cfg, eps, groups = self.cfg, self.cfg["norm"]["eps"], self.cfg["norm"]["groups"]
        T = len(tokens)
        positions = torch.arange(self.pos, self.pos + T)
        x = self.t["embed"][torch.tensor(tokens)]
        for i, L in enumerate(cfg["layers"]):
            h = group_rms(x, self.t[f"l{i}.norm1"], groups, eps)
            p = self.sub(f"l{i}.mix.")
            if L["type"] == "general_delta":
                y = general_delta(h, p, L["mixer"]["heads"], L["mixer"]["dim"], eps, self.state[i])
            elif L["type"] == "latent_attention":
                y = latent_attention(h, p, L["mixer"], eps, positions, self.state[i])
            else:
                raise ValueError(L["type"])
            ml = L.get("mlp")
            if ml:
                q = self.sub(f"l{i}.mlp.")
                if ml["kind"] == "dense":
                    y = y + clamped_glu(h, q["gate"], q["up"], q["down"], ml["limit"])
                elif ml["kind"] == "moe":
                    E = ml["router"]["experts"]
                    ex = [(q[f"e{e}.gate"], q[f"e{e}.up"], q[f"e{e}.down"]) for e in range(E)]
                    y = y + table_moe(h, tokens, q["table"], ex, ml["expert"]["limit"])
                else:
                    raise ValueError(ml["kind"])
            x = x + y
            if layer_outputs is not None:
                layer_outputs.append(x.clone())
        self.pos += T
        z = group_rms(x, self.t["final.norm"], groups, eps) @ self.t["head"].T
        cap = cfg.get("logit_softcap")
        if cap:
            z = cap * torch.tanh(z / cap)
        return z
