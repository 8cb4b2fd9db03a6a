"""Python front end of the tcgen05 GEMM family (`csrc/gemm`).

Naming: `nt` = both operands K-major (`A[M,K] @ B[N,K]^T`), `nn` = B stored
`[K,N]` (MN-major), `tn` = both operands stored with the contraction index as
rows (`A[Kc,M]^T @ B[Kc,N]`).  No operand is ever transposed in memory; the
kernel reads each layout directly through TMA and the tcgen05 descriptors.
"""
from __future__ import annotations

import os

import torch

from . import _ext

MODE_DENSE, MODE_GROUPED_M, MODE_GROUPED_K = 0, 1, 2
EPI_BF16, EPI_F32, EPI_SWIGLU, EPI_SWIGLU_BWD, EPI_LSE, EPI_BF16_SCATTER, EPI_QKROPE = 0, 1, 2, 3, 4, 5, 6

_status_words: dict[int, torch.Tensor] = {}

STATUS_NAMES = {1: "producer wait ran out", 2: "mma wait ran out", 3: "epilogue wait ran out",
                4: "peer wait ran out", 5: "bad argument"}


def status_word(device: torch.device) -> torch.Tensor:
    """Per-device int32 word that kernels write when a bounded wait gives up."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    t = _status_words.get(idx)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", idx))
        _status_words[idx] = t
    return t


def check_status(device: torch.device | None = None) -> None:
    """Synchronising check of the status word; raises if any kernel reported a timeout."""
    devs = [device.index] if device is not None else list(_status_words)
    for idx in devs:
        t = _status_words.get(idx)
        if t is None:
            continue
        v = int(t.item())
        if v != 0:
            t.zero_()
            raise RuntimeError(f"moe_b200 kernel status {v}: {STATUS_NAMES.get(v, 'unknown')}")


def pair_tiles_enabled() -> bool:
    """Pair-tile (`cta_group::2`) kernels are the default; MOE_B200_GEMM_PAIR=0 selects the one-CTA tiles."""
    return os.environ.get("MOE_B200_GEMM_PAIR", "1") != "0"


def _use_pair(M: int, N: int, bn: int | None) -> bool:
    # a pair tile is 256 rows; narrow outputs (router logits) stay on the 64-wide one-CTA tiles
    return pair_tiles_enabled() and M >= 256 and N >= 128 and (bn is None or bn >= 128)


def _pick_bn(n: int) -> int:
    if n <= 64:
        return 64
    if n <= 128:
        return 128
    return 256


def _launch(*, mode, epi, bn, a_mn, b_mn, M, N, K, A, lda, a_inner, a_rows, B, ldb, b_expert_stride, b_inner,
            b_rows, b_experts, C, ldc, num_experts=1, m_fast=1, beta=0, n_half=0, tile_expert=None,
            num_m_tiles=None, seg_off=None, c_expert_stride=0, aux0=None, ld_aux0=0, aux1=None, ld_aux1=0, ep=None,
            cta2=0, pair_tiles=None, a_gather=None, b_gather=None, row_slot=None, row_w=None, row_dot=None,
            rope=None):
    ext = _ext.load()
    ext.gemm(mode, epi, bn, a_mn, b_mn, M, N, K, num_experts, m_fast, beta, n_half, A, lda, a_inner, a_rows, B, ldb,
             b_expert_stride, b_inner, b_rows, b_experts, tile_expert, num_m_tiles, seg_off, C, ldc,
             c_expert_stride, aux0, ld_aux0, aux1, ld_aux1, status_word(A.device), cta2=cta2, pair_tiles=pair_tiles,
             a_gather=a_gather, b_gather=b_gather, row_slot=row_slot, row_w=row_w, row_dot=row_dot, **(rope or {}),
             **(ep or {}))


def _check2d(t: torch.Tensor, name: str) -> None:
    if t.dim() != 2 or t.stride(1) != 1 or t.dtype != torch.bfloat16:
        raise ValueError(f"{name} must be a 2-D bf16 tensor with unit inner stride")
    if t.stride(0) % 8 != 0 or t.data_ptr() % 16 != 0:
        raise ValueError(f"{name}: row pitch must be a multiple of 8 elements and the base 16-byte aligned")


def gemm_nt(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor | None = None, *, out_dtype=torch.bfloat16,
            beta: int = 0, bn: int | None = None, m_fast: int = 1, pair: bool | None = None) -> torch.Tensor:
    """`a[M,K] @ b[N,K]^T` -> `[M,N]` (bf16, or fp32 with optional accumulate)."""
    _check2d(a, "a"); _check2d(b, "b")
    M, K = a.shape
    N = b.shape[0]
    assert b.shape[1] == K
    if out is None:
        out = torch.empty(M, N, dtype=out_dtype, device=a.device)
    epi = EPI_BF16 if out.dtype == torch.bfloat16 else EPI_F32
    pair = (_use_pair(M, N, bn) and (epi == EPI_BF16 or N > 128) and (pair is not False)
            and out.stride(0) % (8 if epi == EPI_BF16 else 4) == 0)
    _launch(mode=MODE_DENSE, epi=epi, bn=(256 if N > 128 else 128) if pair else (bn or _pick_bn(N)), a_mn=0, b_mn=0,
            M=M, N=N, K=K, A=a, lda=a.stride(0), a_inner=K, a_rows=M, B=b, ldb=b.stride(0), b_expert_stride=0,
            b_inner=K, b_rows=N, b_experts=1, C=out, ldc=out.stride(0), beta=beta, m_fast=m_fast, cta2=int(pair))
    return out


def qkv_rope_supported(M: int, N: int, K: int, hd: int) -> bool:
    """Whether the QKV projection can apply the per-head RMSNorm and RoPE in its epilogue (pair-tile kernel,
    head_dim 128: a 256-column tile is two heads).  MOE_B200_QKV_FUSED=0 keeps the separate kernel."""
    return (pair_tiles_enabled() and hd == 128 and M >= 256 and N % 128 == 0 and K % 8 == 0
            and os.environ.get("MOE_B200_QKV_FUSED", "1") != "0")


def gemm_nt_qkrope(a: torch.Tensor, b: torch.Tensor, cs: torch.Tensor, qw: torch.Tensor, kw: torch.Tensor, S: int,
                   nh: int, nkv: int, eps: float) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Fused QKV projection `a[M,K] @ b[N,K]^T` with N = (nh + 2 nkv) * 128.  Returns the raw projection `[M,N]`
    (what backward needs), the same layout with the q / k heads RMS-normalised (fp32 weights `qw`, `kw` `[128]`),
    rotated by the table `cs [S,64,2]` (row r at position r % S) and the v heads copied, and the reciprocal RMS
    `[M, nh + nkv]` of every q / k head."""
    _check2d(a, "a"); _check2d(b, "b")
    M, K = a.shape
    N = b.shape[0]
    raw = torch.empty(M, N, dtype=torch.bfloat16, device=a.device)
    rot = torch.empty(M, N, dtype=torch.bfloat16, device=a.device)
    rstd = torch.empty(M, nh + nkv, dtype=torch.float32, device=a.device)
    _launch(mode=MODE_DENSE, epi=EPI_QKROPE, bn=256, a_mn=0, b_mn=0, M=M, N=N, K=K, A=a, lda=a.stride(0), a_inner=K,
            a_rows=M, B=b, ldb=b.stride(0), b_expert_stride=0, b_inner=K, b_rows=N, b_experts=1, C=raw, ldc=N,
            aux0=rot, ld_aux0=N, cta2=1,
            rope=dict(rope_cs=cs, rope_w=qw, rope_kw=kw, rope_rstd=rstd, rope_S=S, rope_nh=nh, rope_nkv=nkv, rope_eps=eps))
    return raw, rot, rstd


def gemm_nn(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor | None = None, *, bn: int | None = None,
            m_fast: int = 0, pair: bool | None = None) -> torch.Tensor:
    """`a[M,K] @ b[K,N]` -> bf16 `[M,N]`; `b` is read in place (N contiguous)."""
    _check2d(a, "a"); _check2d(b, "b")
    M, K = a.shape
    N = b.shape[1]
    assert b.shape[0] == K
    if out is None:
        out = torch.empty(M, N, dtype=torch.bfloat16, device=a.device)
    pair = _use_pair(M, N, bn) and (pair is not False)
    bn = (128 if N <= 128 else 256) if pair else (bn or (128 if N <= 128 else 256))
    _launch(mode=MODE_DENSE, epi=EPI_BF16, bn=bn, a_mn=0, b_mn=1, M=M, N=N, K=K, A=a, lda=a.stride(0), a_inner=K,
            a_rows=M, B=b, ldb=b.stride(0), b_expert_stride=0, b_inner=N, b_rows=K, b_experts=1, C=out,
            ldc=out.stride(0), m_fast=m_fast, cta2=int(pair))
    return out


_SPLIT_SEG: dict = {}


def _split_k_segments(Kc: int, device) -> torch.Tensor | None:
    """Segment offsets (int32, on the device) that cut a contraction of `Kc` rows into up to 64 equal pieces
    of whole 64-row blocks; None when `Kc` does not divide that way.  Cached: built outside graph capture."""
    key = (Kc, str(device))
    if key not in _SPLIT_SEG:
        blocks = Kc // 64
        parts = 0
        if Kc % 64 == 0:
            parts = max((s for s in range(1, 65) if blocks % s == 0), default=0)
        _SPLIT_SEG[key] = (torch.arange(parts + 1, dtype=torch.int32, device=device) * (Kc // parts)
                           if parts >= 8 else None)
    return _SPLIT_SEG[key]


def gemm_tn(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor, *, beta: int = 0, bn: int | None = None,
            pair: bool | None = None) -> torch.Tensor:
    """`out[M,N] (+)= a[Kc,M]^T @ b[Kc,N]`, fp32 output (weight-gradient shape).  A short, wide output with a long
    contraction (the router's weight gradient: 16 x H over all tokens) has only N / 256 tiles to give to 148 SMs;
    it is cut along the contraction into partial products (one grouped-by-contraction launch) that a fixed-order
    sum then folds into `out`."""
    _check2d(a, "a"); _check2d(b, "b")
    Kc, M = a.shape
    N = b.shape[1]
    assert b.shape[0] == Kc and out.dtype == torch.float32 and out.stride(1) == 1
    if (pair is not False and bn is None and pair_tiles_enabled() and M < 256 and N >= 256 and Kc >= 4096
            and out.is_contiguous() and M * N % 4 == 0):
        seg = _split_k_segments(Kc, a.device)
        if seg is not None:
            S = seg.numel() - 1
            part = torch.empty(S, M, N, dtype=torch.float32, device=a.device)
            _launch(mode=MODE_GROUPED_K, epi=EPI_F32, bn=256, a_mn=1, b_mn=1, M=M, N=N, K=0, A=a, lda=a.stride(0),
                    a_inner=M, a_rows=Kc, B=b, ldb=b.stride(0), b_expert_stride=0, b_inner=N, b_rows=Kc, b_experts=1,
                    C=part, ldc=N, c_expert_stride=M * N, num_experts=S, seg_off=seg, beta=0, m_fast=0, cta2=1)
            _ext.load().sum_partials(part, out, bool(beta))
            return out
    pair = _use_pair(M, N, bn) and out.stride(0) % 4 == 0 and (pair is not False)
    bn = (128 if N <= 128 else 256) if pair else (bn or (128 if N <= 128 else 256))
    _launch(mode=MODE_DENSE, epi=EPI_F32, bn=bn, a_mn=1, b_mn=1, M=M, N=N, K=Kc, A=a, lda=a.stride(0), a_inner=M,
            a_rows=Kc, B=b, ldb=b.stride(0), b_expert_stride=0, b_inner=N, b_rows=Kc, b_experts=1, C=out,
            ldc=out.stride(0), beta=beta, m_fast=0, cta2=int(pair))
    return out


def gemm_nt_lse(a: torch.Tensor, b: torch.Tensor, logits: torch.Tensor | None = None,
                part: torch.Tensor | None = None) -> tuple[torch.Tensor, torch.Tensor]:
    """Vocabulary projection: bf16 logits plus per-(row, 256-column tile) `(max, sum exp)` partials."""
    _check2d(a, "a"); _check2d(b, "b")
    M, K = a.shape
    N = b.shape[0]
    if logits is None:
        logits = torch.empty(M, N, dtype=torch.bfloat16, device=a.device)
    n_tiles = (N + 255) // 256
    if part is None:
        part = torch.empty(M, n_tiles, 2, dtype=torch.float32, device=a.device)
    assert part.shape == (M, n_tiles, 2) and part.is_contiguous()
    _launch(mode=MODE_DENSE, epi=EPI_LSE, bn=256, a_mn=0, b_mn=0, M=M, N=N, K=K, A=a, lda=a.stride(0), a_inner=K,
            a_rows=M, B=b, ldb=b.stride(0), b_expert_stride=0, b_inner=K, b_rows=N, b_experts=1, C=logits,
            ldc=logits.stride(0), aux0=part, m_fast=1, cta2=int(_use_pair(M, N, 256)))
    return logits, part


# ------------------------------------------------------------------ dense SwiGLU MLP
def dense_up_swiglu(x: torch.Tensor, w_gate_up: torch.Tensor, act: torch.Tensor, gu: torch.Tensor) -> None:
    """`x[T,H]` x `w_gate_up[2I,H]` (gate rows, then up rows) -> `act[T,I] = silu(gate) * up`, `gu[T,2I]`."""
    _check2d(x, "x"); _check2d(w_gate_up, "w_gate_up")
    T, H = x.shape
    I = w_gate_up.shape[0] // 2
    pair = _use_pair(T, 2 * I, None)
    _launch(mode=MODE_DENSE, epi=EPI_SWIGLU, bn=256, a_mn=0, b_mn=0, M=T, N=I, K=H, A=x, lda=x.stride(0), a_inner=H,
            a_rows=T, B=w_gate_up, ldb=w_gate_up.stride(0), b_expert_stride=0, b_inner=H, b_rows=2 * I, b_experts=1,
            C=act, ldc=act.stride(0), n_half=I, aux0=gu, ld_aux0=gu.stride(0), m_fast=0, cta2=int(pair))


def dense_swiglu_bwd(dy: torch.Tensor, w_down: torch.Tensor, gu: torch.Tensor, dgu: torch.Tensor) -> None:
    """`d(act) = dy[T,H] @ w_down[H,I]` fused with the SwiGLU backward: writes `dgu[T,2I]`."""
    _check2d(dy, "dy"); _check2d(w_down, "w_down")
    T, H = dy.shape
    I = w_down.shape[1]
    pair = _use_pair(T, I, None) and I > 128
    _launch(mode=MODE_DENSE, epi=EPI_SWIGLU_BWD, bn=256 if I > 128 else 128, a_mn=0, b_mn=1, M=T, N=I, K=H, A=dy,
            lda=dy.stride(0), a_inner=H, a_rows=T, B=w_down, ldb=w_down.stride(0), b_expert_stride=0, b_inner=I,
            b_rows=H, b_experts=1, C=dgu, ldc=dgu.stride(0), n_half=I, aux0=gu, ld_aux0=gu.stride(0), aux1=dgu,
            ld_aux1=dgu.stride(0), m_fast=0, cta2=int(pair))


# ------------------------------------------------------------------ grouped (MoE)
def _pair_kw(pair, N: int) -> dict:
    """Arguments that switch a grouped-by-rows GEMM to the pair-tile kernel.  `pair` = (pair_tiles int32
    [P, 2], num_pair_tiles int32 [1]) from the dispatch plan, or None."""
    if pair is None or not pair_tiles_enabled() or N < 128:
        return {}
    return dict(cta2=1, pair_tiles=pair[0], num_m_tiles=pair[1], bn=256)


def fold_supported(H: int, I2: int) -> bool:
    """Whether the routing weight can be applied inside the expert GEMMs' epilogues (pair-tile kernels)."""
    return (pair_tiles_enabled() and I2 > 256 and H > 128 and H % 8 == 0
            and os.environ.get("MOE_B200_MOE_FOLD", "1") != "0")


def gather_supported(H: int, I2: int) -> bool:
    """Whether the expert GEMMs fetch token rows by index (TMA gather in the pair-tile kernels) instead of
    reading a materialised expert-sorted copy.  Off unless MOE_B200_MOE_GATHER=1: a `tile::gather4` copy moves
    four 128-byte rows, and at 32 of them per 16 KB operand tile the copy engine, not the tensor pipe, bounds the
    main loop (the gathered GEMMs measured 3 to 4 times slower than the same GEMMs on a sorted copy)."""
    return fold_supported(H, I2) and os.environ.get("MOE_B200_MOE_GATHER", "0") == "1"


def grouped_up_swiglu(xs: torch.Tensor, w_gate_up: torch.Tensor, tile_expert: torch.Tensor,
                      num_m_tiles: torch.Tensor, act: torch.Tensor, gu: torch.Tensor, bn: int = 256, ep=None,
                      pair=None, gather: torch.Tensor | None = None, row_slot=None, row_w=None) -> None:
    """`xs[R,H]` (expert-sorted, 128-row padded) x `w_gate_up[E,2I,H]` -> `act[R,I]`, pre-activations `gu[R,2I]`.
    With `gather` (int32, one source row per sorted row; pair-tile kernel only) `xs` is the UNSORTED `[T,H]`
    activation and the kernel's producer fetches row `gather[r]` for sorted row r: dispatch is the A-operand load."""
    H = xs.shape[1]
    R = act.shape[0]
    E, I2, _ = w_gate_up.shape
    I = I2 // 2
    kw = dict(bn=bn, num_m_tiles=num_m_tiles)
    kw.update(_pair_kw(pair, 2 * I))
    if gather is not None:
        if not kw.get("cta2"):
            raise ValueError("row gather needs the pair-tile kernel")
        kw["a_gather"] = gather
    if row_w is not None:  # routing weight folded into the stored activation
        kw.update(row_slot=row_slot, row_w=row_w)
    _launch(mode=MODE_GROUPED_M, epi=EPI_SWIGLU, a_mn=0, b_mn=0, M=R, N=I, K=H, A=xs, lda=xs.stride(0),
            a_inner=H, a_rows=xs.shape[0], B=w_gate_up, ldb=w_gate_up.stride(1), b_expert_stride=w_gate_up.stride(0),
            b_inner=H, b_rows=I2, b_experts=E, C=act, ldc=act.stride(0), n_half=I, tile_expert=tile_expert,
            aux0=gu, ld_aux0=gu.stride(0), m_fast=0, ep=ep, **kw)


def grouped_nt(xs: torch.Tensor, w: torch.Tensor, tile_expert: torch.Tensor, num_m_tiles: torch.Tensor,
               out: torch.Tensor, bn: int | None = None, ep=None, scatter: bool = False, pair=None) -> None:
    """`out[R,N] = xs[R,K] @ w[e(row)][N,K]^T` (down projection).  `scatter=True`: rows go to the peers'
    return buffers named in `ep` instead of `out` (only `out.stride(0)` is used)."""
    R, K = xs.shape
    E, N, _ = w.shape
    kw = dict(bn=bn or (128 if N <= 128 else 256), num_m_tiles=num_m_tiles)
    if not scatter:
        kw.update(_pair_kw(pair, N))
    _launch(mode=MODE_GROUPED_M, epi=EPI_BF16_SCATTER if scatter else EPI_BF16, a_mn=0, b_mn=0, M=R, N=N, K=K,
            A=xs, lda=xs.stride(0), a_inner=K, a_rows=R, B=w, ldb=w.stride(1), b_expert_stride=w.stride(0),
            b_inner=K, b_rows=N, b_experts=E, C=out, ldc=out.stride(0), tile_expert=tile_expert,
            m_fast=0, ep=ep, **kw)


def grouped_nn(xs: torch.Tensor, w: torch.Tensor, tile_expert: torch.Tensor, num_m_tiles: torch.Tensor,
               out: torch.Tensor, bn: int | None = None, ep=None, scatter: bool = False, pair=None) -> None:
    """`out[R,N] = xs[R,K] @ w[e(row)][K,N]` (input gradients; weights read in place)."""
    R, K = xs.shape
    E, _, N = w.shape
    kw = dict(bn=bn or (128 if N <= 128 else 256), num_m_tiles=num_m_tiles)
    if not scatter:
        kw.update(_pair_kw(pair, N))
    _launch(mode=MODE_GROUPED_M, epi=EPI_BF16_SCATTER if scatter else EPI_BF16, a_mn=0, b_mn=1, M=R, N=N, K=K,
            A=xs, lda=xs.stride(0), a_inner=K, a_rows=R, B=w, ldb=w.stride(1), b_expert_stride=w.stride(0),
            b_inner=N, b_rows=K, b_experts=E, C=out, ldc=out.stride(0), tile_expert=tile_expert,
            m_fast=0, ep=ep, **kw)


def grouped_nn_swiglu_bwd(dy: torch.Tensor, w_down: torch.Tensor, tile_expert: torch.Tensor,
                          num_m_tiles: torch.Tensor, gu: torch.Tensor, dgu: torch.Tensor,
                          bn: int | None = None, ep=None, pair=None, gather: torch.Tensor | None = None,
                          row_slot=None, row_w=None, row_dot=None) -> None:
    """`d(act) = dy[R,H] @ w_down[e][H,I]`, fused with the SwiGLU backward: writes `dgu[R,2I]`.  With `gather`
    `dy` is the unsorted `[T,H]` output gradient and sorted row r reads `dy[gather[r]]`; `row_w` / `row_slot`
    multiply the incoming gradient by the routing weight and `row_dot [R, ceil(I/256)]` receives the partial
    dot products that make up the routing-weight gradient."""
    H = dy.shape[1]
    R = dgu.shape[0]
    E, _, I = w_down.shape
    kw = dict(bn=bn or (128 if I <= 128 else 256), num_m_tiles=num_m_tiles)
    kw.update(_pair_kw(pair, I if I > 128 else 0))
    if gather is not None or row_w is not None:
        if not kw.get("cta2"):
            raise ValueError("row gather / weight folding need the pair-tile kernel")
        kw.update(a_gather=gather, row_slot=row_slot, row_w=row_w, row_dot=row_dot)
    _launch(mode=MODE_GROUPED_M, epi=EPI_SWIGLU_BWD, a_mn=0, b_mn=1, M=R, N=I,
            K=H, A=dy, lda=dy.stride(0), a_inner=H, a_rows=dy.shape[0], B=w_down, ldb=w_down.stride(1),
            b_expert_stride=w_down.stride(0), b_inner=I, b_rows=H, b_experts=E, C=dgu, ldc=dgu.stride(0),
            n_half=I, tile_expert=tile_expert, aux0=gu, ld_aux0=gu.stride(0), aux1=dgu,
            ld_aux1=dgu.stride(0), m_fast=0, ep=ep, **kw)


def grouped_tn(a: torch.Tensor, b: torch.Tensor, seg_off: torch.Tensor, out: torch.Tensor, beta: int = 0,
               bn: int | None = None, b_gather: torch.Tensor | None = None,
               a_gather: torch.Tensor | None = None) -> None:
    """Per-expert weight gradient: `out[e][M,N] (+)= a[seg_e, M]^T @ b[seg_e, N]`, fp32.  With `b_gather` (int32
    per sorted row) `b` is the unsorted `[T,N]` tensor and contraction row k reads `b[b_gather[k]]`."""
    R, M = a.shape
    N = b.shape[1]
    E = out.shape[0]
    pair = _use_pair(M, N, bn) and out.stride(1) % 4 == 0 and out.stride(0) % 4 == 0
    if (b_gather is not None and not (pair and N > 128)) or (a_gather is not None and not pair):
        raise ValueError("row gather needs the 256-wide pair-tile kernel")
    _launch(mode=MODE_GROUPED_K, epi=EPI_F32, bn=(128 if N <= 128 else 256) if pair else (bn or (128 if N <= 128 else 256)),
            a_mn=1, b_mn=1, M=M, N=N, K=0,
            A=a, lda=a.stride(0), a_inner=M, a_rows=a.shape[0], B=b, ldb=b.stride(0), b_expert_stride=0, b_inner=N,
            b_rows=b.shape[0], b_experts=1, C=out, ldc=out.stride(1), c_expert_stride=out.stride(0), num_experts=E,
            seg_off=seg_off, beta=beta, m_fast=0, cta2=int(pair), b_gather=b_gather, a_gather=a_gather)
