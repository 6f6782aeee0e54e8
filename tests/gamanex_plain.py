"""Plain float64 restatement of the Gamanex design, one function per mechanism, for the tests. It shares no code with the engine.

A model is (cfg, weights): cfg is the config.json tree, weights maps tensor names to torch tensors. Notation: x [T, W] is the residual
stream of T tokens of one sequence (positions 0 .. T-1), h a normed copy of it.

  layer:      x <- x + ls1 * sigmoid(rg1 h1 + b1) * mixer(h1) + ls2 * sigmoid(rg2 h2 + b2) * ff(h2),  h1 = rms(x) * n1, h2 = rms(x) * n2
  attention:  q = rms_all(Wq h1) * wq * temp(p),  k = rms_all(Wk h1) * wk,  v = Wv h1
              s[i, j] = scale * q_i . k_j - r1 * ln(1 + r2 * (i - j)) + pb   (per head),  j <= i
              out_i = sum_j sigmoid(s[i, j]) * v_j                              (no normalisation over j)
  ff dense:   Wd relu(Wu h2)^2
  ff experts: logits = Wr h2 + br; the `top` largest; weights = softmax over those; sum_e weight_e * Wd_e (silu(Wg_e h2) * (Wu_e h2))
  readout:    logit_scale * head (rms(x) * final.norm)
"""
import math

import torch

F64 = torch.float64


def rms_norm(x, w, eps):
    x = x.to(F64)
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps) * w.to(F64)


def query_temperature(positions, coef, every):
    """1 + coef * ln(floor((p + 1) / every) + 1)"""
    p = torch.as_tensor(positions, dtype=torch.int64)
    return 1.0 + coef * torch.log((torch.div(p + 1, every, rounding_mode="floor") + 1).to(F64))


def distance_bias(r1, r2, dist):
    """r1 * ln(1 + r2 * dist), per head: r1, r2 [H], dist [...] -> [H, ...]"""
    d = dist.to(F64)
    shape = (-1,) + (1,) * d.dim()
    return r1.to(F64).reshape(shape) * torch.log1p(r2.to(F64).reshape(shape) * d)


def sigmoid_attention(q, k, v, positions_q, positions_k, heads, kv_heads, dim, vdim, scale, r1, r2, pb):
    """q [Tq, heads*dim], k [Tk, kv_heads*dim], v [Tk, kv_heads*vdim] -> [Tq, heads*vdim]. Key j is visible to query i when pos_k[j] <= pos_q[i]."""
    Tq, Tk = q.shape[0], k.shape[0]
    q = q.to(F64).reshape(Tq, heads, dim)
    k = k.to(F64).reshape(Tk, kv_heads, dim)
    v = v.to(F64).reshape(Tk, kv_heads, vdim)
    per = heads // kv_heads
    pq = torch.as_tensor(positions_q, dtype=torch.int64)
    pk = torch.as_tensor(positions_k, dtype=torch.int64)
    dist = pq[:, None] - pk[None, :]
    visible = dist >= 0
    bias = distance_bias(r1, r2, dist.clamp(min=0))            # [H, Tq, Tk]
    out = torch.zeros(Tq, heads, vdim, dtype=F64)
    for h in range(heads):
        g = h // per
        s = (q[:, h, :] @ k[:, g, :].T) * scale - bias[h] + float(pb[h])
        w = torch.sigmoid(s) * visible
        out[:, h, :] = w @ v[:, g, :]
    return out.reshape(Tq, heads * vdim)


def attention_keys_values(h, W, prefix, eps):
    """The cached part of an attention layer that owns its keys: k after the whole-projection norm, and v."""
    k = h @ W[prefix + "mix.k"].to(F64).T
    k = rms_norm(k, W[prefix + "mix.k.norm"], eps)
    v = h @ W[prefix + "mix.v"].to(F64).T
    return k, v


def attention_mixer(h, W, prefix, mc, eps, positions, kv):
    """h [T, width] at `positions`; kv = (k, v, positions_k) of every visible token (this layer's own or another layer's)."""
    q = h @ W[prefix + "mix.q"].to(F64).T
    q = rms_norm(q, W[prefix + "mix.q.norm"], eps)
    qt = mc.get("q_temp")
    if qt:
        q = q * query_temperature(positions, qt["coef"], qt["every"])[:, None]
    k, v, pk = kv
    o = sigmoid_attention(q, k, v, positions, pk, mc["heads"], mc["kv_heads"], mc["dim"], mc["vdim"], mc["scale"],
                          W[prefix + "mix.r1"], W[prefix + "mix.r2"], W[prefix + "mix.pb"])
    return o @ W[prefix + "mix.o"].to(F64).T


def dense_ff(h, W, prefix):
    u = torch.relu(h @ W[prefix + "mlp.up"].to(F64).T)
    return (u * u) @ W[prefix + "mlp.down"].to(F64).T


def route(h, W, prefix, top):
    """-> (indices [T, top], weights [T, top]): the largest logits (the lower index wins a tie), softmax over the chosen ones"""
    z = h @ W[prefix + "mlp.router"].to(F64).T + W[prefix + "mlp.router.b"].to(F64)
    order = torch.sort(z, dim=-1, descending=True, stable=True).indices[:, :top]
    return order, torch.softmax(torch.gather(z, 1, order), dim=-1)


def expert_ff(h, W, prefix):
    g = h @ W[prefix + "gate"].to(F64).T
    u = h @ W[prefix + "up"].to(F64).T
    return (g * torch.sigmoid(g) * u) @ W[prefix + "down"].to(F64).T


def moe_ff(h, W, prefix, ml):
    idx, wt = route(h, W, prefix, ml["router"]["top"])
    out = torch.zeros(h.shape[0], W[prefix + "mlp.e0.down"].shape[0], dtype=F64)
    for e in range(ml["router"]["experts"]):
        rows, slots = torch.nonzero(idx == e, as_tuple=True)
        if len(rows):
            out[rows] += wt[rows, slots][:, None] * expert_ff(h[rows], W, f"{prefix}mlp.e{e}.")
    return out


def sublayer_gate(h, W, name):
    return torch.sigmoid(h @ W[name].to(F64).T + W[name + ".b"].to(F64))


def forward(cfg, W, tokens, layer_outputs=None):
    """Logits [T, vocab] of one sequence fed whole. layer_outputs: a list that receives the residual stream after every layer."""
    eps = cfg["norm"]["eps"]
    T = len(tokens)
    pos = list(range(T))
    x = W["embed"].to(F64)[torch.as_tensor(tokens, dtype=torch.int64)]
    kv = {}
    for i, lc in enumerate(cfg["layers"]):
        p = f"l{i}."
        mc = lc["mixer"]
        if lc["type"] != "attention":
            raise ValueError("unknown layer type " + lc["type"])
        h1 = rms_norm(x, W[p + "norm1"], eps)
        src = mc.get("kv_from")
        if src is None:
            k, v = attention_keys_values(h1, W, p, eps)
            kv[i] = (k, v, pos)
            src = i
        y = attention_mixer(h1, W, p, mc, eps, pos, kv[src])
        y = y * W[p + "ls1"].to(F64) * sublayer_gate(h1, W, p + "rg1")
        ml = lc.get("mlp")
        if ml:
            h2 = rms_norm(x, W[p + "norm2"], eps)
            f = dense_ff(h2, W, p) if ml["kind"] == "dense" else moe_ff(h2, W, p, ml)
            y = y + f * W[p + "ls2"].to(F64) * sublayer_gate(h2, W, p + "rg2")
        x = x + y
        if layer_outputs is not None:
            layer_outputs.append(x.clone())
    return (rms_norm(x, W["final.norm"], eps) @ W["head"].to(F64).T) * cfg.get("logit_scale", 1.0)


# ---- random models ---------------------------------------------------------------------------------------------------------------
def attention_layer(heads, kv_heads, dim, vdim, scale=None, q_temp=None, kv_from=None, mlp=None):
    mc = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale if scale is not None else 1.0 / math.sqrt(dim)}
    if q_temp:
        mc["q_temp"] = {"coef": q_temp[0], "every": q_temp[1]}
    if kv_from is not None:
        mc["kv_from"] = kv_from
    return {"type": "attention", "mixer": mc, "mlp": mlp}


def dense_mlp(ff):
    return {"kind": "dense", "ff": ff}


def moe_mlp(ff, experts, top):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def make_config(width, vocab, layers, eps=1e-5, logit_scale=0.5):
    return {"architecture": "Gamanex", "width": width, "vocab": vocab, "norm": {"eps": eps}, "logit_scale": logit_scale, "layers": layers}


def random_weights(cfg, seed=0, dtype=torch.bfloat16):
    """Weights in the checkpoint's layout, values exactly representable in `dtype`."""
    g = torch.Generator().manual_seed(seed)
    Wd, V = cfg["width"], cfg["vocab"]
    out = {}

    def mat(name, rows, cols, gain=1.0):
        out[name] = (torch.randn(rows, cols, generator=g) * gain / math.sqrt(cols)).to(dtype)

    def vec(name, n, mean=0.0, std=1.0, positive=False):
        t = torch.randn(n, generator=g) * std + mean
        out[name] = (t.abs() + 0.05 if positive else t).to(dtype)

    out["embed"] = torch.randn(V, Wd, generator=g).to(dtype)
    mat("head", V, Wd)
    vec("final.norm", Wd, 1.0, 0.1)
    for i, lc in enumerate(cfg["layers"]):
        p = f"l{i}."
        mc = lc["mixer"]
        H, G, D, Dv = mc["heads"], mc["kv_heads"], mc["dim"], mc["vdim"]
        vec(p + "norm1", Wd, 1.0, 0.1)
        mat(p + "mix.q", H * D, Wd)
        vec(p + "mix.q.norm", H * D, 1.0, 0.2)
        if mc.get("kv_from") is None:
            mat(p + "mix.k", G * D, Wd)
            mat(p + "mix.v", G * Dv, Wd)
            vec(p + "mix.k.norm", G * D, 1.0, 0.2)
        vec(p + "mix.r1", H, 0.5, 0.3, positive=True)
        vec(p + "mix.r2", H, 0.3, 0.2, positive=True)
        vec(p + "mix.pb", H, -1.0, 0.5)
        mat(p + "mix.o", Wd, H * Dv)
        vec(p + "ls1", Wd, 0.7, 0.2)
        mat(p + "rg1", Wd, Wd)
        vec(p + "rg1.b", Wd, 0.3, 0.5)
        ml = lc.get("mlp")
        if ml:
            vec(p + "norm2", Wd, 1.0, 0.1)
            vec(p + "ls2", Wd, 0.7, 0.2)
            mat(p + "rg2", Wd, Wd)
            vec(p + "rg2.b", Wd, 0.3, 0.5)
            if ml["kind"] == "dense":
                mat(p + "mlp.up", ml["ff"], Wd, 1.5)
                mat(p + "mlp.down", Wd, ml["ff"])
            else:
                E, Fe = ml["router"]["experts"], ml["expert"]["ff"]
                mat(p + "mlp.router", E, Wd, 2.0)
                vec(p + "mlp.router.b", E, 0.0, 0.5)
                for x in range(E):
                    mat(f"{p}mlp.e{x}.gate", Fe, Wd, 1.5)
                    mat(f"{p}mlp.e{x}.up", Fe, Wd, 1.5)
                    mat(f"{p}mlp.e{x}.down", Wd, Fe)
    return out
