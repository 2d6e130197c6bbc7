"""Plain, slow implementation of the Llama dense GQA decoder: whole sequences, no cache.

Every function restates one formula of the reference C++ engine (llm-engine) and cites the
file:line it was read from. It shares no code with the package under test: it parses config.json
and the safetensors file itself, runs on the CPU in float32 (RoPE set-up in float64 as the
reference does) and recomputes every position of a sequence from scratch.

It was compared once with the reference's own compiled model code on tiny random models; the
outputs of that comparison and the script that made them are in tests/golden/.
"""
from __future__ import annotations

import json
import math
import os
import struct

import numpy as np

F32 = np.float32


# ----------------------------------------------------------------------------- checkpoint reading
def read_config(model_dir: str) -> dict:
    """Keys and defaults of load_config (src/weights.cpp:55-121)."""
    with open(os.path.join(model_dir, "config.json")) as f:
        j = json.load(f)
    c = {}
    c["hidden_size"] = j.get("hidden_size", 0)
    c["intermediate_size"] = j.get("intermediate_size", 0)
    c["num_hidden_layers"] = j.get("num_hidden_layers", 0)
    c["num_attention_heads"] = j.get("num_attention_heads", 0)
    c["num_key_value_heads"] = j.get("num_key_value_heads", c["num_attention_heads"])
    c["head_dim"] = j.get("head_dim", c["hidden_size"] // c["num_attention_heads"])
    c["vocab_size"] = j.get("vocab_size", 0)
    c["max_position_embeddings"] = j.get("max_position_embeddings", 0)
    c["rms_norm_eps"] = F32(j.get("rms_norm_eps", 1e-5))
    c["tie_word_embeddings"] = bool(j.get("tie_word_embeddings", False))
    c["rope_theta"] = F32(j.get("rope_theta", 10000.0))  # float field: include/llmengine/config.hpp:19
    c["rope_has_scaling"] = False
    c["rope_factor"] = F32(1.0)
    c["rope_low_freq_factor"] = F32(1.0)
    c["rope_high_freq_factor"] = F32(1.0)
    c["rope_original_max_pos"] = 0

    def scaling(rs):  # src/weights.cpp:79-85
        c["rope_has_scaling"] = True
        c["rope_factor"] = F32(rs.get("factor", 1.0))
        c["rope_low_freq_factor"] = F32(rs.get("low_freq_factor", 1.0))
        c["rope_high_freq_factor"] = F32(rs.get("high_freq_factor", 1.0))
        c["rope_original_max_pos"] = int(rs.get("original_max_position_embeddings", 0))

    if j.get("rope_parameters") is not None:  # src/weights.cpp:87-96
        rp = j["rope_parameters"]
        c["rope_theta"] = F32(rp.get("rope_theta", c["rope_theta"]))
        if rp.get("rope_type", "default") == "llama3":
            scaling(rp)
    elif j.get("rope_scaling") is not None:
        scaling(j["rope_scaling"])

    eos = set()  # src/weights.cpp:98-118

    def absorb(src):
        e = src.get("eos_token_id")
        if isinstance(e, list):
            eos.update(int(v) for v in e)
        elif isinstance(e, int):
            eos.add(e)

    absorb(j)
    gen = os.path.join(model_dir, "generation_config.json")
    if os.path.exists(gen):
        with open(gen) as f:
            absorb(json.load(f))
    c["eos_token_ids"] = eos
    return c


def read_safetensors(path: str) -> dict:
    """u64 header length, JSON header, data section (src/weights.cpp:170-241).
    Every tensor is widened to float32: bf16 by bits<<16 (src/model.cpp:14-40)."""
    with open(path, "rb") as f:
        raw = f.read()
    (hlen,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + hlen])
    data = memoryview(raw)[8 + hlen:]
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        b, e = meta["data_offsets"]
        buf = bytes(data[b:e])
        dt = meta["dtype"]
        if dt == "F32":
            a = np.frombuffer(buf, dtype="<f4").astype(F32)
        elif dt == "BF16":
            a = (np.frombuffer(buf, dtype="<u2").astype(np.uint32) << 16).view(F32)
        elif dt == "F16":
            a = np.frombuffer(buf, dtype="<f2").astype(F32)
        else:
            raise ValueError(f"plain reader: dtype {dt} of {name}")
        out[name] = a.reshape(meta["shape"]).copy()
    return out


def read_model(model_dir: str):
    cfg = read_config(model_dir)
    w = {}
    for fn in sorted(os.listdir(model_dir)):  # src/weights.cpp:37-51
        if fn.endswith(".safetensors"):
            w.update(read_safetensors(os.path.join(model_dir, fn)))
    if cfg["tie_word_embeddings"]:  # src/weights.cpp:244-267
        w["lm_head.weight"] = w["model.embed_tokens.weight"]
    return cfg, w


# ----------------------------------------------------------------------------- parts
def embed(table: np.ndarray, ids) -> np.ndarray:
    """out = E[id,:] (src/kernels.cpp:59-66)."""
    return table[np.asarray(ids, dtype=np.int64)].astype(F32)


def rmsnorm(x: np.ndarray, w: np.ndarray, eps) -> np.ndarray:
    """sumsq in float32; inv = 1/sqrt(sumsq/dim + eps); out = w*x*inv (src/kernels.cpp:18-24)."""
    x = x.astype(F32)
    ss = np.sum(x * x, axis=-1, keepdims=True, dtype=F32)
    inv = F32(1.0) / np.sqrt(ss / F32(x.shape[-1]) + F32(eps), dtype=F32)
    return (w.astype(F32) * x) * inv


def linear(x: np.ndarray, w: np.ndarray) -> np.ndarray:
    """out[m,n] = sum_k x[m,k]*w[n,k], W row-major [N,K], no bias (src/kernels.cpp:33-57)."""
    return (x.astype(F32) @ w.astype(F32).T).astype(F32)


def silu(x: np.ndarray) -> np.ndarray:
    """v/(1+exp(-v)) (src/kernels.cpp:26-31)."""
    x = x.astype(F32)
    return x / (F32(1.0) + np.exp(-x, dtype=F32))


def swiglu_mlp(x, w_gate, w_up, w_down) -> np.ndarray:
    """g=Wg x; u=Wu x; g=silu(g); g*=u; out=Wd g (src/engine.cpp:383-412)."""
    g = silu(linear(x, w_gate))
    g = g * linear(x, w_up)
    return linear(g, w_down)


_PI_F32 = float(F32(3.14159265358979323846))  # the float constant kPi (src/kernels.cpp:110-112)


def llama3_inv_freq(head_dim, theta, has_scaling, factor, low_f, high_f, orig_max_pos) -> np.ndarray:
    """float64 theta^(-2i/hd) with the Llama-3 wavelength bands, rounded to float32
    (src/kernels.cpp:114-160)."""
    half = head_dim // 2
    theta = float(theta)
    inv = [1.0 / math.pow(theta, (2 * i) / head_dim) for i in range(half)]
    if has_scaling:
        factor, low_f, high_f = float(factor), float(low_f), float(high_f)
        low_wl = orig_max_pos / low_f
        high_wl = orig_max_pos / high_f
        band = high_f - low_f
        two_pi = 2.0 * _PI_F32
        for i in range(half):
            fr = inv[i]
            wl = two_pi / fr
            if wl > low_wl:
                inv[i] = fr / factor
            elif wl < high_wl:
                pass
            else:
                smooth = (orig_max_pos / wl - low_f) / band
                inv[i] = (1.0 - smooth) * fr / factor + smooth * fr
    return np.array(inv, dtype=np.float64).astype(F32)


def rope_tables(inv_freq_f32: np.ndarray, max_pos: int, head_dim: int):
    """angle = double(p)*double(inv_freq_f32[i]); cos/sin cast to float32; halves duplicated
    (src/kernels.cpp:162-187)."""
    ang = np.arange(max_pos, dtype=np.float64)[:, None] * inv_freq_f32.astype(np.float64)[None, :]
    c = np.cos(ang).astype(F32)
    s = np.sin(ang).astype(F32)
    return np.concatenate([c, c], axis=1), np.concatenate([s, s], axis=1)


def apply_rope(x: np.ndarray, cos_rows: np.ndarray, sin_rows: np.ndarray) -> np.ndarray:
    """x [T, heads, hd]; per head: x[i]=a*cos[i]-b*sin[i]; x[i+h]=b*cos[i+h]+a*sin[i+h]
    (src/kernels.cpp:189-203)."""
    half = x.shape[-1] // 2
    a = x[..., :half]
    b = x[..., half:]
    c = cos_rows[:, None, :]
    s = sin_rows[:, None, :]
    return np.concatenate([a * c[..., :half] - b * s[..., :half],
                           b * c[..., half:] + a * s[..., half:]], axis=-1).astype(F32)


def causal_gqa_attention(q: np.ndarray, k: np.ndarray, v: np.ndarray) -> np.ndarray:
    """q [T,nq,hd], k/v [T,nkv,hd] -> [T,nq*hd]. Query t sees keys 0..t. kv head = h // (nq/nkv);
    score = dot * (1/sqrt(hd)) (scale after the dot); p = exp(s-max); p *= 1/sum; o = sum p*V
    (src/kernels.cpp:413-474; causal range from src/engine.cpp:358-362)."""
    T, nq, hd = q.shape
    nkv = k.shape[1]
    g = nq // nkv
    scale = F32(1.0) / np.sqrt(F32(hd))
    out = np.zeros((T, nq, hd), dtype=F32)
    for h in range(nq):
        kv = h // g
        s = (q[:, h, :] @ k[:, kv, :].T).astype(F32) * scale  # [T, T]
        mask = np.tril(np.ones((T, T), dtype=bool))
        s = np.where(mask, s, F32(-np.inf))
        m = s.max(axis=1, keepdims=True)
        p = np.exp(s - m, dtype=F32)
        inv = F32(1.0) / p.sum(axis=1, keepdims=True, dtype=F32)
        p = p * inv
        out[:, h, :] = p @ v[:, kv, :]
    return out.reshape(T, nq * hd)


def attention_block(x, cfg, w, layer: int, cos, sin) -> np.ndarray:
    """q/k/v projections, RoPE on q and k at absolute positions, attention, o projection
    (src/engine.cpp:319-379)."""
    T = x.shape[0]
    nq, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    p = f"model.layers.{layer}.self_attn."
    q = linear(x, w[p + "q_proj.weight"]).reshape(T, nq, hd)
    k = linear(x, w[p + "k_proj.weight"]).reshape(T, nkv, hd)
    v = linear(x, w[p + "v_proj.weight"]).reshape(T, nkv, hd)
    q = apply_rope(q, cos[:T], sin[:T])
    k = apply_rope(k, cos[:T], sin[:T])
    a = causal_gqa_attention(q, k, v)
    return linear(a, w[p + "o_proj.weight"])


def position_limit(cfg) -> int:
    """The engine under test serves positions up to max_position_embeddings; the reference caps
    its table at min(max_pos, original_max_pos, 8192) (include/llmengine/config.hpp:39-45), a
    limit of its table size only: the angle formula is the same at every position."""
    return int(cfg["max_position_embeddings"])


def forward_logits(cfg, w, ids) -> np.ndarray:
    """Logits [T,V] at every position of one sequence (src/engine.cpp:694-716 with the layer loop
    of src/engine.cpp:105-261): h=E[id]; per layer h+=Attn(RMSNorm(h)); h+=MLP(RMSNorm(h));
    logits = lm_head(RMSNorm(h))."""
    return logits_at(cfg, w, final_hidden(cfg, w, ids), None)


def logits_at(cfg, w, h: np.ndarray, rows) -> np.ndarray:
    """Final norm and head for the given rows of the residual stream (all rows if None): the
    reference skips both for positions whose logits are not asked for (src/engine.cpp:415-433)."""
    x = rmsnorm(h if rows is None else h[np.asarray(rows, dtype=np.int64)], w["model.norm.weight"], cfg["rms_norm_eps"])
    return linear(x, w["lm_head.weight"])


def final_hidden(cfg, w, ids) -> np.ndarray:
    """The residual stream [T,H] after the last layer (the layer loop of src/engine.cpp:105-261)."""
    T = len(ids)
    hd = cfg["head_dim"]
    inv = llama3_inv_freq(hd, cfg["rope_theta"], cfg["rope_has_scaling"], cfg["rope_factor"],
                          cfg["rope_low_freq_factor"], cfg["rope_high_freq_factor"],
                          cfg["rope_original_max_pos"])
    cos, sin = rope_tables(inv, T, hd)
    eps = cfg["rms_norm_eps"]
    h = embed(w["model.embed_tokens.weight"], ids)
    for l in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{l}."
        x = rmsnorm(h, w[p + "input_layernorm.weight"], eps)
        h = h + attention_block(x, cfg, w, l, cos, sin)
        x = rmsnorm(h, w[p + "post_attention_layernorm.weight"], eps)
        h = h + swiglu_mlp(x, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"],
                           w[p + "mlp.down_proj.weight"])
    return h


# ----------------------------------------------------------------------------- sampling, generation
def argmax_first(row: np.ndarray) -> int:
    """First index of the maximum, strict '>' (src/engine.cpp:52-58)."""
    return int(np.argmax(row))


def _mix32(x: np.ndarray) -> np.ndarray:
    x = x.astype(np.uint32)
    x ^= x >> np.uint32(16)
    x = (x * np.uint32(0x7FEB352D)).astype(np.uint32)
    x ^= x >> np.uint32(15)
    x = (x * np.uint32(0x846CA68B)).astype(np.uint32)
    x ^= x >> np.uint32(16)
    return x


def gumbel_noise(seed: int, draw_index: int, n: int) -> np.ndarray:
    """The engine's counter-based noise (no counterpart in the reference, which samples greedily
    only): u_i from a 32-bit integer hash of (seed, draw_index, i); g_i = -log(-log(u_i))."""
    with np.errstate(over="ignore"):
        i = np.arange(n, dtype=np.uint32)
        k = _mix32(np.full(n, seed & 0xFFFFFFFF, dtype=np.uint32) ^ np.uint32(0x9E3779B9))
        k = _mix32(k + np.uint32(draw_index & 0xFFFFFFFF))
        r = _mix32(k ^ (i * np.uint32(0x85EBCA6B)).astype(np.uint32))
    u = ((r >> np.uint32(9)).astype(F32) + F32(0.5)) * F32(1.0 / 8388608.0)
    return -np.log(-np.log(u, dtype=F32), dtype=F32)


def sample_token(row: np.ndarray, temperature: float, seed: int, draw_index: int) -> int:
    """temperature 0: greedy. Else argmax_i(logit_i/T + g_i): a draw from softmax(logits/T)."""
    if temperature <= 0.0:
        return argmax_first(row)
    z = row.astype(F32) * (F32(1.0) / F32(temperature)) + gumbel_noise(seed, draw_index, row.shape[0])
    return int(np.argmax(z))


def generate(cfg, w, prompt, max_new_tokens, temperature=0.0, seed=0):
    """Greedy loop of Engine::generate (src/engine.cpp:718-774) by re-running the whole sequence:
    EOS is not appended ("stop"); else "length". draw_index = number of tokens generated so far."""
    out = list(prompt)
    finish = "length"
    while len(out) - len(prompt) < max_new_tokens:
        logits = forward_logits(cfg, w, out)[-1]
        nxt = sample_token(logits, temperature, seed, len(out) - len(prompt))
        if nxt in cfg["eos_token_ids"]:
            finish = "stop"
            break
        out.append(nxt)
    return out, finish
