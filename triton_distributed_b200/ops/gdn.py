"""Gated DeltaNet (gated delta rule linear attention), forward.

API of the reference: ``chunk_gated_delta_rule_fwd(q, k, v, g, beta, scale, initial_state, output_final_state,
cu_seqlens)`` -> ``(g_cumsum, o, A, final_state)`` (python/triton_dist/kernels/nvidia/gdn.py:926-970); inputs are
``[1, T, H, K|V]`` with several sequences packed along T and delimited by ``cu_seqlens``.

Per head the state ``S`` [K, V] follows ``S <- exp(g_t) S;  v' = beta_t (v_t - S^T k_t);  S <- S + k_t v'^T;
o_t = scale S^T q_t``.  Three implementations of the same function live here:

* ``csrc/gdn_chunk.cu``: the chunk-parallel WY form the reference uses (triangular solve per 64-token chunk,
  sequential pass over chunk states, output pass) as three CUDA kernels with tensor-core products - the default for
  bf16 CUDA tensors with K = 128 and V a multiple of 64, also the source of the per-chunk ``A`` matrices;
* ``csrc/gdn.cu``: one CUDA kernel that walks the tokens with the state in registers (``impl="recurrent"``; other V);
* ``gated_delta_rule_chunked``: the same chunked form with batched PyTorch ops - the CPU path;
* ``gated_delta_rule_recurrent``: the token loop in fp32, the oracle of the tests.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from .. import _native

CHUNK = 64


def prepare_lens(cu_seqlens: torch.Tensor) -> torch.Tensor:
    return cu_seqlens[1:] - cu_seqlens[:-1]


def prepare_chunk_indices(cu_seqlens: torch.Tensor, chunk_size: int = CHUNK) -> torch.Tensor:
    """(sequence index, chunk index inside the sequence) of every chunk, as the reference's helper (gdn.py:56-60)."""
    lens = prepare_lens(cu_seqlens).tolist()
    idx = [(s, c) for s, n in enumerate(lens) for c in range((n + chunk_size - 1) // chunk_size)]
    return torch.tensor(idx, dtype=torch.int32, device=cu_seqlens.device).reshape(-1, 2)


def gated_delta_rule_recurrent(q, k, v, g, beta, scale, initial_state=None, cu_seqlens=None):
    """Token-by-token fp32 reference.  q, k [1, T, H, K]; v [1, T, H, V]; g, beta [1, T, H].  Returns (o, final_state)."""
    _, T, H, K = q.shape
    V = v.shape[-1]
    cu = [0, T] if cu_seqlens is None else cu_seqlens.tolist()
    o = torch.zeros(1, T, H, V, dtype=torch.float32, device=q.device)
    states = []
    for s in range(len(cu) - 1):
        S = (initial_state[s].float().clone() if initial_state is not None
             else torch.zeros(H, K, V, dtype=torch.float32, device=q.device))
        for t in range(cu[s], cu[s + 1]):
            kt, qt, vt = k[0, t].float(), q[0, t].float(), v[0, t].float()
            S = S * torch.exp(g[0, t].float())[:, None, None]
            r = torch.einsum("hkv,hk->hv", S, kt)
            vn = beta[0, t].float()[:, None] * (vt - r)
            S = S + kt[:, :, None] * vn[:, None, :]
            o[0, t] = torch.einsum("hkv,hk->hv", S, qt) * scale
        states.append(S)
    return o, torch.stack(states)


def gated_delta_rule_chunked(q, k, v, g, beta, scale, initial_state=None, cu_seqlens=None, chunk: int = CHUNK):
    """Chunk-parallel form (fp32 math): returns (g_cumsum, o, A, final_state) like the reference's entry point."""
    _, T, H, K = q.shape
    V = v.shape[-1]
    dev = q.device
    cu = [0, T] if cu_seqlens is None else cu_seqlens.tolist()
    o = torch.zeros(1, T, H, V, dtype=torch.float32, device=dev)
    gc_all = torch.zeros(1, T, H, dtype=torch.float32, device=dev)
    A_all = torch.zeros(1, T, H, chunk, dtype=torch.float32, device=dev)
    finals = []
    for s in range(len(cu) - 1):
        a, b = cu[s], cu[s + 1]
        n = b - a
        nc = (n + chunk - 1) // chunk
        pad = nc * chunk - n

        def prep(x, fill=0.0):
            x = x[0, a:b].float()
            if pad:
                x = torch.cat([x, torch.full((pad,) + x.shape[1:], fill, dtype=x.dtype, device=dev)], 0)
            return x.reshape(nc, chunk, *x.shape[1:]).transpose(1, 2) if x.dim() == 3 else x.reshape(nc, chunk, H).transpose(1, 2)

        qc, kc, vc = prep(q), prep(k), prep(v)                       # [nc, H, C, *]
        gcs = prep(g).cumsum(-1)                                     # [nc, H, C] chunk-local cumulative log decay
        bc = prep(beta)
        # A = (I + tril(beta K K^T * exp(g_i - g_j), -1))^-1, then w = A (beta k exp(g)), u = A (beta v)
        decay = torch.exp((gcs[..., :, None] - gcs[..., None, :]).tril())
        kk = torch.einsum("nhik,nhjk->nhij", kc * bc[..., None], kc) * decay
        L = torch.eye(chunk, device=dev) + kk.tril(-1)
        A = torch.linalg.solve_triangular(L, torch.eye(chunk, device=dev).expand_as(L), upper=False)
        w = A @ (kc * (bc * torch.exp(gcs))[..., None])
        u = A @ (vc * bc[..., None])
        S = (initial_state[s].float().clone() if initial_state is not None
             else torch.zeros(H, K, V, dtype=torch.float32, device=dev))
        causal = torch.ones(chunk, chunk, device=dev).tril().bool()
        outs = []
        for c in range(nc):
            g_c = gcs[c]                                             # [H, C]
            v_new = u[c] - w[c] @ S                                  # [H, C, V]
            attn = (qc[c] @ kc[c].transpose(-1, -2)) * torch.exp(g_c[:, :, None] - g_c[:, None, :]).masked_fill(~causal, 0)
            outs.append(((qc[c] * torch.exp(g_c)[..., None]) @ S + attn.masked_fill(~causal, 0) @ v_new) * scale)
            g_last = g_c[:, -1]
            S = S * torch.exp(g_last)[:, None, None] + (kc[c] * torch.exp(g_last[:, None] - g_c)[..., None]).transpose(-1, -2) @ v_new
        # padded rows carry g = 0, beta = 0, k = 0: they neither change the state nor the outputs of real rows
        oc = torch.stack(outs, 0).transpose(1, 2).reshape(nc * chunk, H, V)[:n]
        o[0, a:b] = oc
        gc_all[0, a:b] = gcs.transpose(1, 2).reshape(nc * chunk, H)[:n]
        A_all[0, a:b] = A.transpose(1, 2).reshape(nc * chunk, H, chunk)[:n]
        finals.append(S)
    return gc_all, o, A_all, torch.stack(finals)


def chunk_gated_delta_rule_fwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, g: torch.Tensor, beta: torch.Tensor,
                               scale: float, initial_state: Optional[torch.Tensor] = None,
                               output_final_state: bool = False, cu_seqlens: Optional[torch.Tensor] = None,
                               return_A: bool = False, impl: str = "auto") -> Tuple[torch.Tensor, torch.Tensor, Optional[torch.Tensor], Optional[torch.Tensor]]:
    """Forward of the gated delta rule.  Returns ``(g_cumsum, o, A, final_state)``: the chunk-local cumulative log
    decay, the outputs in the dtype of ``v``, the per-chunk WY matrices (only with ``return_A``; otherwise None) and the
    final state fp32 [N, H, K, V] (with ``output_final_state``).  ``impl``: "auto" (chunk-parallel CUDA kernels where they
    apply, else the token-recurrent kernel, else PyTorch), "chunk" or "recurrent"."""
    _, T, H, K = q.shape
    V = v.shape[-1]
    if cu_seqlens is None:
        cu_seqlens = torch.tensor([0, T], dtype=torch.int32, device=q.device)
    native = _native.use_native(q, k, v) and q.dtype == torch.bfloat16 and K == 128
    chunk_ok = native and V % 64 == 0 and 64 <= V <= 256 and impl in ("auto", "chunk")
    recurrent_ok = native and V % 32 == 0 and not return_A and impl in ("auto", "recurrent")
    if impl == "chunk" and not chunk_ok or impl == "recurrent" and not recurrent_ok:
        raise ValueError(f"chunk_gated_delta_rule_fwd: impl={impl!r} does not support these tensors")
    if chunk_ok:
        lib = _native.load(True)
        cu = cu_seqlens.to(device=q.device, dtype=torch.int32).contiguous()
        chunk_seq, chunk_t0, seq_chunk0 = _chunk_tables(cu_seqlens, q.device)
        o, gc, A, ht = lib.gdn_chunk_fwd(q[0].contiguous(), k[0].contiguous(), v[0].contiguous(), g[0].float().contiguous(),
                                         beta[0].to(torch.bfloat16).contiguous(), float(scale),
                                         initial_state.float().contiguous() if initial_state is not None else None,
                                         bool(output_final_state), cu, chunk_seq, chunk_t0, seq_chunk0, bool(return_A))
        return gc.unsqueeze(0), o.unsqueeze(0), (A.unsqueeze(0) if return_A else None), (ht if output_final_state else None)
    if not recurrent_ok:
        gc, o, A, ht = gated_delta_rule_chunked(q, k, v, g, beta, scale, initial_state, cu_seqlens)
        return gc, o.to(v.dtype), (A if return_A else None), (ht if output_final_state else None)
    lib = _native.load(True)
    cu = cu_seqlens.to(device=q.device, dtype=torch.int32)
    o, ht = lib.gdn_fwd(q[0].contiguous(), k[0].contiguous(), v[0].contiguous(), g[0].float().contiguous(),
                        beta[0].to(torch.bfloat16).contiguous(), float(scale),
                        initial_state.float().contiguous() if initial_state is not None else None,
                        bool(output_final_state), cu)
    # chunk-local cumulative decay, cheap enough in torch: cumsum over T minus the value at each chunk start
    gc = _chunk_local_cumsum(g[0].float(), cu_seqlens)
    return gc.unsqueeze(0), o.unsqueeze(0), None, (ht if output_final_state else None)


def _chunk_tables(cu_seqlens: torch.Tensor, device, chunk: int = CHUNK):
    """Per chunk: its sequence and first token; per sequence: its first chunk (int32 device tensors)."""
    cu = cu_seqlens.tolist()
    seq_of, t0_of, first = [], [], [0]
    for s in range(len(cu) - 1):
        for t in range(cu[s], cu[s + 1], chunk):
            seq_of.append(s)
            t0_of.append(t)
        first.append(len(seq_of))
    mk = lambda x: torch.tensor(x, dtype=torch.int32, device=device)   # noqa: E731
    return mk(seq_of), mk(t0_of), mk(first)


def _chunk_local_cumsum(g: torch.Tensor, cu_seqlens: torch.Tensor, chunk: int = CHUNK) -> torch.Tensor:
    out = torch.empty_like(g)
    cu = cu_seqlens.tolist()
    for s in range(len(cu) - 1):
        a, b = cu[s], cu[s + 1]
        n = b - a
        nc = (n + chunk - 1) // chunk
        pad = nc * chunk - n
        x = g[a:b]
        if pad:
            x = torch.cat([x, x.new_zeros(pad, x.shape[1])], 0)
        out[a:b] = x.reshape(nc, chunk, -1).cumsum(1).reshape(nc * chunk, -1)[:n]
    return out
