"""Helpers shared by the GPU parity tests (not a test module)."""
import numpy as np
import torch

from oracle import c_oracle, kv_oracle

TOL = {torch.float32: dict(rtol=1e-4, atol=1e-5), torch.bfloat16: dict(rtol=0.0, atol=2e-2)}


def to_oracle(t: torch.Tensor) -> np.ndarray:
    """Device tensor -> numpy array the C oracle takes (fp32 as is, bf16 as uint16 bits)."""
    t = t.detach().contiguous().cpu()
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().view(np.uint16)
    return t.numpy()


def to_f32(t: torch.Tensor) -> np.ndarray:
    return t.detach().to(torch.float32).cpu().numpy()


def randn(shape, dtype, device, seed):
    """Seeded N(0,1) values drawn on `device` (fast for large caches), rounded to `dtype`."""
    g = torch.Generator(device=device).manual_seed(seed)
    return torch.randn(shape, generator=g, dtype=torch.float32, device=device).to(dtype)


def make_ctx(pkg):
    return pkg.gpu.context_create(0)


def buf2d(pkg, ctx, t: torch.Tensor):
    """Wrap an existing 2-D device tensor as a GPUBuffer2D."""
    return pkg.gpu.GPUBuffer2D(buffer=t, shape=tuple(t.shape), size=t.numel())


def logical_view(cache, layer, which):
    """[B, T_max, H, D] torch view/copy of a contiguous (non-paged) cache, by plain indexing."""
    buf = (layer.k_cache if which == "k" else layer.v_cache).buffer
    B, T, H, D = cache.batch_size, cache.max_seq_len, cache.n_heads, cache.head_dim
    if cache.layout == "bthd":
        return buf.reshape(B, T, H, D)
    return buf.reshape(B, H, T, D).permute(0, 2, 1, 3)


def oracle_decode(q, k_logical, v_logical, lens):
    """C oracle on the logical [B, T, H, D] arrays (reference layout strides)."""
    B, T, H, D = k_logical.shape
    return c_oracle.decode(to_oracle(q), to_oracle(k_logical), to_oracle(v_logical), np.asarray(lens, dtype=np.int32),
                           B, H, D, (T * H * D, H * D, D))


def fill_cache_logical(cache, layer_idx, k_logical, v_logical):
    """Write logical [B, T, H, D] contents into a cache of any layout with torch indexing
    (test set-up only; the append kernel is tested separately)."""
    layer = cache.layers[layer_idx]
    B, T, H, D = k_logical.shape
    for which, src in (("k", k_logical), ("v", v_logical)):
        buf = (layer.k_cache if which == "k" else layer.v_cache).buffer
        if cache.block_table is not None:
            bs = cache.block_size
            pool = buf.reshape(cache.n_blocks, H, bs, D)
            table = cache.block_table.cpu()
            nb = (T + bs - 1) // bs
            for b in range(B):
                for j in range(nb):
                    cnt = min(bs, T - j * bs)
                    pool[int(table[b, j]), :, :cnt, :] = src[b, j * bs : j * bs + cnt].permute(1, 0, 2)
        elif cache.layout == "bthd":
            buf.reshape(cache.batch_size, cache.max_seq_len, H, D)[:, :T] = src
        else:
            buf.reshape(cache.batch_size, H, cache.max_seq_len, D)[:, :, :T] = src.permute(0, 2, 1, 3)
