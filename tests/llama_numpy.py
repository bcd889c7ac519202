"""Independent float64/float32 numpy Llama forward (textbook formulation, no catgrad op stream): used to check that
the restated Llama term computes a Llama, separately from the oracle/GPU comparison which shares the term."""
import numpy as np


def rmsnorm(x, g, eps):
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps) * g


def llama3_inv_freq(inv, scaling):
    """The frequency rescaling of Llama 3.1 (as published with the model: frequencies whose wavelength exceeds
    original/low_freq_factor are divided by `factor`, those below original/high_freq_factor are kept, linear blend of
    the two in between), in float64."""
    factor, lo, hi = scaling["factor"], scaling["low_freq_factor"], scaling["high_freq_factor"]
    orig = scaling["original_max_position_embeddings"]
    wavelen = 2 * np.pi / inv
    smooth = (orig / wavelen - lo) / (hi - lo)
    blended = (1 - smooth) * inv / factor + smooth * inv
    out = np.where(wavelen > orig / lo, inv / factor, inv)
    mid = (wavelen <= orig / lo) & (wavelen >= orig / hi)
    return np.where(mid, blended, out)


def rope(x, pos0, theta, scaling=None):
    # x [B, h, S, D]; rotate-half convention
    d = x.shape[-1]
    inv = 1.0 / theta ** (np.arange(d // 2, dtype=np.float64) * 2.0 / d)
    if scaling is not None:
        inv = llama3_inv_freq(inv, scaling)
    ang = (pos0 + np.arange(x.shape[2], dtype=np.float64))[:, None] * inv[None, :]
    c = np.concatenate([np.cos(ang), np.cos(ang)], -1)
    s = np.concatenate([np.sin(ang), np.sin(ang)], -1)
    rot = np.concatenate([-x[..., d // 2:], x[..., :d // 2]], -1)
    return x * c + rot * s


def forward(cfg, w, ids, cache=None):
    """ids [B, S] -> logits [B, S, V] (float64); cache = list of (k, v) per layer or None."""
    w = {k: v.astype(np.float64) for k, v in w.items()}
    b, s = ids.shape
    nh, nkv, hd = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    x = w["model.embed_tokens.weight"][ids]
    pos0 = 0 if cache is None else cache[0][0].shape[2]
    new_cache = []
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        h = rmsnorm(x, w[p + "input_layernorm.weight"], cfg.rms_norm_eps)
        q = (h @ w[p + "self_attn.q_proj.weight"].T).reshape(b, s, nh, hd).transpose(0, 2, 1, 3)
        k = (h @ w[p + "self_attn.k_proj.weight"].T).reshape(b, s, nkv, hd).transpose(0, 2, 1, 3)
        v = (h @ w[p + "self_attn.v_proj.weight"].T).reshape(b, s, nkv, hd).transpose(0, 2, 1, 3)
        scaling = getattr(cfg, "rope_scaling", None)
        q, k = rope(q, pos0, cfg.rope_theta, scaling), rope(k, pos0, cfg.rope_theta, scaling)
        if cache is not None:
            k = np.concatenate([cache[i][0], k], 2)
            v = np.concatenate([cache[i][1], v], 2)
        new_cache.append((k, v))
        kk, vv = np.repeat(k, nh // nkv, 1), np.repeat(v, nh // nkv, 1)
        sc = q @ kk.transpose(0, 1, 3, 2) / np.sqrt(hd)
        t = k.shape[2]
        mask = np.arange(t)[None, :] > (pos0 + np.arange(s))[:, None]
        sc = np.where(mask, -np.inf, sc)
        sc = np.exp(sc - sc.max(-1, keepdims=True))
        pr = sc / sc.sum(-1, keepdims=True)
        a = (pr @ vv).transpose(0, 2, 1, 3).reshape(b, s, nh * hd)
        x = x + a @ w[p + "self_attn.o_proj.weight"].T
        h = rmsnorm(x, w[p + "post_attention_layernorm.weight"], cfg.rms_norm_eps)
        g = h @ w[p + "mlp.gate_proj.weight"].T
        u = h @ w[p + "mlp.up_proj.weight"].T
        x = x + ((g / (1 + np.exp(-g))) * u) @ w[p + "mlp.down_proj.weight"].T
    x = rmsnorm(x, w["model.norm.weight"], cfg.rms_norm_eps)
    head = w["model.embed_tokens.weight"] if cfg.tie_word_embeddings else w["lm_head.weight"]
    return x @ head.T, new_cache
