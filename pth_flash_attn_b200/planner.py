"""Host-side launch planner of ``pth_flash_attn_fwd`` for B200 (sm_100a).

Same public surface as the reference planner (python/pth_flash_attn/planner.py:
``plan_launch``, ``LaunchPlan``, ``c_target``, ``s_alone``, ``max_tokens_per_tile``,
``wm_for_rows``, ``split_tile_range``, ``workspace_token_splits``,
``workspace_shapes``, ``workspace_bytes``, ``DESCRIPTOR_FIELDS``), same contract:

* pure Python, standard library only, no device query;
* every input is a host ``int``/``bool`` of the padded batch descriptor (a 0-d
  tensor is refused: converting it would be a hidden device-to-host sync);
* there is no sequence-length parameter, so a plan is valid for every replay of
  a CUDA graph captured for its descriptor.

What differs is the machine model.  A row tile of this library holds up to 64
rows (query heads of one KV head x query tokens), as in the reference, but at
head size 128 the kernel is one warp-specialised CTA per SM (it keeps about
220 KB of cache bytes in flight in shared memory) on a 148-SM part and reads
the cache in 128-key tiles.  The split count is chosen per launch from the
descriptor:

    work items per split = Hkv * row tiles            (row tiles: see below)
    S = max(1, C_target // items)

that is: no split once the unsplit work items fill the GPU, otherwise the
largest count that still fits ONE wave.  Every CTA pays a fixed cost (finding
its row tile, quantising Q, filling the copy pipeline, merging its two softmax
groups) worth some tens of KV tiles, and every split adds a partial for the
combine kernel to read, so more, shorter CTAs than one wave lose more than a
fuller last wave wins (measured on B200 at 8 K and 128 K keys per request).
``wm`` keeps its meaning of "16 * wm rows per tile" because it is part of the
op's frozen schema; the kernels pad rows to 16/32/64 accordingly.
"""

from __future__ import annotations

from dataclasses import dataclass

ROWS_PER_WM = 16
WM_CHOICES = (1, 2, 4)
MAX_ROWS_PER_CTA = ROWS_PER_WM * WM_CHOICES[-1]
# Resident CTAs per SM of the attention kernels, by head size.
CTAS_PER_SM = {64: 4, 128: 1, 256: 2}
SUPPORTED_HEAD_SIZES = tuple(sorted(CTAS_PER_SM))
WINDOWED_HEAD_SIZES = (128,)
KV_TILE_TOKENS = 128
PARTIAL_BYTES_PER_ELEMENT = 4
B200_NUM_SMS = 148

DESCRIPTOR_FIELDS = (
    "num_tokens",
    "num_reqs",
    "max_query_len",
    "G",
    "Hkv",
    "D",
    "num_sms",
    "is_prefill",
    "ws_token_splits",
    "window",
)


def _ceil_div(a: int, b: int) -> int:
    return -(-a // b)


def _require_int(name: str, value: object, minimum: int) -> int:
    if not isinstance(value, int) or isinstance(value, bool):
        raise TypeError(f"{name} must be a host int, got {type(value).__name__}")
    if value < minimum:
        raise ValueError(f"{name} must be >= {minimum}, got {value}")
    return value


def _require_head_size(D: object) -> int:
    d = _require_int("D", D, 1)
    if d not in CTAS_PER_SM:
        raise ValueError(f"D must be one of {SUPPORTED_HEAD_SIZES}, got {d}")
    return d


def _require_group_size(G: object) -> int:
    g = _require_int("G", G, 1)
    if g > MAX_ROWS_PER_CTA:
        raise ValueError(f"G must be <= {MAX_ROWS_PER_CTA}, got {g}")
    return g


def c_target(*, D: int, num_sms: int) -> int:
    """CTAs that fill the GPU in one wave: SMs x resident CTAs per SM at head size D."""
    d = _require_head_size(D)
    return _require_int("num_sms", num_sms, 1) * CTAS_PER_SM[d]


def max_tokens_per_tile(G: int) -> int:
    """Query tokens of one request that fit one 64-row tile: ``64 // G``."""
    return MAX_ROWS_PER_CTA // _require_group_size(G)


def wm_for_rows(rows: int) -> int:
    """Smallest wm in {1, 2, 4} with ``16 * wm >= rows``."""
    r = _require_int("rows", rows, 1)
    for wm in WM_CHOICES:
        if r <= ROWS_PER_WM * wm:
            return wm
    raise ValueError(f"{r} rows exceed one {MAX_ROWS_PER_CTA}-row tile")


def split_tile_range(*, split: int, num_splits: int, num_tiles: int) -> tuple[int, int]:
    """KV tiles ``[floor(s T / S), floor((s + 1) T / S))`` of split ``s`` (the device rule)."""
    s_count = _require_int("num_splits", num_splits, 1)
    s = _require_int("split", split, 0)
    tiles = _require_int("num_tiles", num_tiles, 0)
    if s >= s_count:
        raise ValueError(f"split {s} out of range for num_splits={s_count}")
    return s * tiles // s_count, (s + 1) * tiles // s_count


@dataclass(frozen=True)
class LaunchPlan:
    """What one ``pth_flash_attn_fwd`` call needs from the host.

    ``wm`` and ``num_splits`` are arguments of the op; the other fields record
    the descriptor and the shapes derived from it.
    """

    wm: int
    bq: int
    q_tiles_upper: int
    num_splits: int
    num_tokens: int
    G: int
    Hkv: int
    D: int
    is_prefill: bool

    @property
    def Hq(self) -> int:
        return self.G * self.Hkv

    @property
    def rows_per_cta(self) -> int:
        return self.bq * self.G

    @property
    def grid(self) -> tuple[int, int, int]:
        return (self.q_tiles_upper, self.Hkv, self.num_splits)

    @property
    def ws_token_splits_used(self) -> int:
        return self.num_splits * self.num_tokens if self.num_splits > 1 else 0

    @property
    def ws_o_shape(self) -> tuple[int, int, int, int]:
        s = self.num_splits if self.num_splits > 1 else 0
        return (s, self.num_tokens, self.Hq, self.D)

    @property
    def ws_lse_shape(self) -> tuple[int, int, int]:
        s = self.num_splits if self.num_splits > 1 else 0
        return (s, self.num_tokens, self.Hq)


def _pick_splits(items: int, target: int) -> int:
    """Largest split count whose CTAs still fit one wave (1 if the items alone fill it)."""
    return max(1, target // items)


def plan_launch(
    *,
    num_tokens: int,
    num_reqs: int,
    max_query_len: int,
    G: int,
    Hkv: int,
    D: int,
    num_sms: int,
    is_prefill: bool,
    ws_token_splits: int,
    window: int = 0,
) -> LaunchPlan:
    """Plan one launch from the padded batch descriptor of its slice."""
    t = _require_int("num_tokens", num_tokens, 1)
    reqs = _require_int("num_reqs", num_reqs, 1)
    q_max = _require_int("max_query_len", max_query_len, 1)
    g = _require_group_size(G)
    hkv = _require_int("Hkv", Hkv, 1)
    d = _require_head_size(D)
    sms = _require_int("num_sms", num_sms, 1)
    w_ts = _require_int("ws_token_splits", ws_token_splits, 0)
    w = _require_int("window", window, 0)
    if not isinstance(is_prefill, bool):
        raise TypeError(f"is_prefill must be a bool, got {type(is_prefill).__name__}")
    if q_max > t:
        raise ValueError(f"max_query_len={q_max} > num_tokens={t}")
    if t > reqs * q_max:
        raise ValueError(f"num_tokens={t} cannot come from {reqs} requests of at most {q_max} tokens")

    b_max = max_tokens_per_tile(g)
    if is_prefill:
        wm = WM_CHOICES[-1]
        row_tiles = _ceil_div(t, b_max)
    else:
        rt = _ceil_div(q_max, b_max)
        wm = wm_for_rows(_ceil_div(q_max, rt) * g)
        # every request is assumed to bring its full rt tiles (lengths are not visible here)
        row_tiles = rt * reqs
    bq = ROWS_PER_WM * wm // g

    s_want = _pick_splits(hkv * row_tiles, c_target(D=d, num_sms=sms))
    s_cap = w_ts // t
    num_splits = max(1, min(s_want, s_cap))
    if w > 0:
        # The most KV tiles one row tile can touch at the worst alignment.
        num_splits = min(num_splits, _ceil_div(w + q_max - 2, KV_TILE_TOKENS) + 1)

    return LaunchPlan(
        wm=wm,
        bq=bq,
        q_tiles_upper=t // bq + reqs,
        num_splits=num_splits,
        num_tokens=t,
        G=g,
        Hkv=hkv,
        D=d,
        is_prefill=is_prefill,
    )


def s_alone(*, Hkv: int, D: int, num_sms: int) -> int:
    """Splits that let ONE row tile per KV head fill one wave of the GPU."""
    hkv = _require_int("Hkv", Hkv, 1)
    return _pick_splits(hkv, c_target(D=D, num_sms=num_sms))


def workspace_token_splits(*, max_num_seqs: int, q_dec_max: int, Hkv: int, D: int, num_sms: int) -> int:
    """Token-splits to reserve so that every plan this module makes fits.

    A launch of R requests of up to ``q_dec_max`` tokens needs ``S * T`` with
    ``T <= R * q_dec_max`` and ``S <= max(1, C_target // (Hkv * R))``.
    """
    seqs = _require_int("max_num_seqs", max_num_seqs, 1)
    q_dec = _require_int("q_dec_max", q_dec_max, 1)
    alone = s_alone(Hkv=Hkv, D=D, num_sms=num_sms)
    target = c_target(D=D, num_sms=num_sms)
    hkv = _require_int("Hkv", Hkv, 1)
    worst = 0
    for r in range(1, seqs + 1):
        worst = max(worst, min(_pick_splits(hkv * r, target), alone) * r * q_dec)
    return worst


def workspace_shapes(*, ws_token_splits: int, Hq: int, D: int) -> tuple[tuple[int, int, int], tuple[int, int]]:
    """fp32 shapes to reserve: O partials ``[W_ts, Hq, D]`` and log2-LSE ``[W_ts, Hq]``."""
    w_ts = _require_int("ws_token_splits", ws_token_splits, 0)
    hq = _require_int("Hq", Hq, 1)
    d = _require_head_size(D)
    return (w_ts, hq, d), (w_ts, hq)


def workspace_bytes(*, ws_token_splits: int, Hq: int, D: int) -> int:
    """``W_ts * Hq * (D + 1) * 4``: both fp32 partial buffers."""
    o_shape, lse_shape = workspace_shapes(ws_token_splits=ws_token_splits, Hq=Hq, D=D)
    return (o_shape[0] * o_shape[1] * o_shape[2] + lse_shape[0] * lse_shape[1]) * PARTIAL_BYTES_PER_ELEMENT
