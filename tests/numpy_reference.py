"""An independent float64 numpy statement of paged attention, used to pin the C
oracle.  It follows the reference's software path step for step
(crates/mlx-sys/src/mlx.cpp:4080-4156): take the sequence's blocks, transpose
{1,0,2,3,4} then {0,1,3,2,4} (K) / {1,0,2,3} then {0,1,3,2} (V), reshape to
[Hkv, nb*BS, D], slice to the context, map query head -> kv head by integer
division, scores*scale, softmax, @V.  Multi-token sequences add the causal limit
kv_len - q_len + j + 1.  It shares no index arithmetic with oracle/paged_oracle.c."""
import numpy as np

from pa_testlib import D, X, elems_to_f32


def gather_sequence(k_pool, v_pool, table_row, kv_len, f16=False):
    BS = v_pool.shape[3]  # tokens per pool block
    D = v_pool.shape[2]   # head size
    nb = (kv_len + BS - 1) // BS
    blocks = table_row[:nb]
    k = k_pool[blocks]                                  # [nb, Hkv, D/X, BS, X]
    k = k.transpose(1, 0, 2, 3, 4).transpose(0, 1, 3, 2, 4)  # [Hkv, nb, BS, D/X, X]
    k = k.reshape(k.shape[0], nb * BS, D)[:, :kv_len]
    v = v_pool[blocks]                                  # [nb, Hkv, D, BS]
    v = v.transpose(1, 0, 2, 3).transpose(0, 1, 3, 2)   # [Hkv, nb, BS, D]
    v = v.reshape(v.shape[0], nb * BS, D)[:, :kv_len]
    return elems_to_f32(np.ascontiguousarray(k), f16).astype(np.float64), \
        elems_to_f32(np.ascontiguousarray(v), f16).astype(np.float64)


def paged_attention(q_bits, k_pool, v_pool, block_tables, kv_lens, cu_q, Hq, Hkv, scale,
                    softcap=1.0, f16=False):
    q = elems_to_f32(q_bits, f16).astype(np.float64)
    out = np.zeros(q.shape, dtype=np.float64)
    G = Hq // Hkv
    for s in range(len(kv_lens)):
        kv_len = int(kv_lens[s])
        q0, q1 = int(cu_q[s]), int(cu_q[s + 1])
        if kv_len == 0 or q1 == q0:
            continue
        k, v = gather_sequence(k_pool, v_pool, block_tables[s], kv_len, f16)
        for j in range(q1 - q0):
            n = kv_len - (q1 - q0) + j + 1
            if n <= 0:
                continue
            for hq in range(Hq):
                h = hq // G
                logits = (k[h, :n] @ q[q0 + j, hq]) * scale
                if softcap != 1.0:
                    logits = np.tanh(logits / softcap) * softcap
                w = np.exp(logits - logits.max())
                out[q0 + j, hq] = (w / w.sum()) @ v[h, :n]
    return out


def qk_norm_rope(x_bits, weight_bits, eps, positions, rope_base, rope_dims, f16=False):
    """Independent numpy statement of the producer (RMS norm per head, then rotary
    embedding with traditional = false, scale 1; crates/mlx-sys/src/mlx.cpp:1343-1365
    applied to one token per sequence at its own offset,
    crates/mlx-core/src/transformer/attention.rs:658-664), vectorised over tokens and
    heads, float64 inside, the 16-bit rounding points of MLX's kernels kept.  Returns the
    rotated values as float64 rounded to the 16-bit type."""
    def rnd(a):
        a32 = a.astype(np.float32)
        if f16:
            return a32.astype(np.float16).astype(np.float64)
        u = a32.view(np.uint32).astype(np.uint64)
        r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint32) << 16
        return r.astype(np.uint32).view(np.float32).astype(np.float64)

    x = elems_to_f32(x_bits, f16).astype(np.float64)          # [T, H, D]
    if weight_bits is not None:
        w = elems_to_f32(weight_bits, f16).astype(np.float64)
        inv = 1.0 / np.sqrt((x * x).mean(axis=-1, keepdims=True) + eps)
        x = rnd(rnd(x * inv) * w)
    half = rope_dims // 2
    inv_freq = np.power(np.float64(rope_base), -np.arange(half) / half).astype(np.float32)
    theta = (np.asarray(positions, dtype=np.float32)[:, None] * inv_freq[None, :]).astype(np.float64)
    c, s_ = np.cos(theta)[:, None, :], np.sin(theta)[:, None, :]
    a, b = x[..., :half], x[..., half:2 * half]
    out = x.copy()
    out[..., :half] = a * c - b * s_
    out[..., half:2 * half] = a * s_ + b * c
    return rnd(out)
