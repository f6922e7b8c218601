"""Host-side launch planner of ``pth_flash_attn_fwd`` for B200 (sm_100a).

The public names, keyword-only signatures, ``DESCRIPTOR_FIELDS`` and exception types are
those of the reference planner (python/pth_flash_attn/planner.py:102-113, 147-381;
docs/api.md:135-145), so callers and their tests can switch modules.  The contract is the
reference's too: pure Python, no device query, every argument a host ``int`` / ``bool``
taken from the padded batch descriptor (a 0-d tensor is refused because converting it
would be a hidden device-to-host copy), and no argument that carries a sequence length,
so one plan is valid for every replay of a CUDA graph captured for its descriptor.

What is planned differs, because the kernels differ:

* The attention kernel for short row tiles is persistent: it is launched with one CTA per
  SM, cuts every request into pieces of about equal length ON THE DEVICE (where the
  lengths are) and deals the pieces out to its CTAs.  The host's ``num_splits`` is
  therefore only a bound - the most pieces a request may be cut into, which is what sizes
  the workspace - and the planner's job is to make that bound generous enough:

      unsplit = Hkv * row tiles of the launch        work items without any split
      S = ceil(ITEMS_PER_SM * SMs / unsplit)         room for the device's choice (it aims at 8 items per SM)
      S = min(S, s_alone)                            never more than a lone request needs

  ``s_alone`` = ``ceil(2 * SMs / Hkv)``: a single request is cut so that every SM gets two
  pieces of it.  The kernel never uses more pieces than keep a piece above a few KV tiles,
  so for this kernel a generous bound costs workspace, not time.
* ``wm`` keeps its meaning of "16 * wm rows per tile" because it is an argument of the
  op's frozen schema; rows per tile are 16, 32 or 64 and the kernels pad to those.
* A sliding window caps the pieces at the number of 128-key tiles a row tile can touch.
* Tall row tiles (more than 16 rows) run on the row-major kernels, which launch one CTA per
  (row tile, KV head, piece of the bound): there a generous bound does cost time - CTAs of
  unused pieces that start only to leave, fp32 partials and a combine for requests the
  device left whole (a drafter step of 32 requests: 183 us at a bound of 10, 146 us at 1).
  Under a sliding window every request longer than the window holds the same work per row
  tile, so pieces only serve to fill the SMs: the bound of a tall windowed launch is
  ``ceil(SMs / unsplit)``.  Without a window the lengths may differ by orders of magnitude
  and the bound stays generous.
"""

from __future__ import annotations

import dataclasses
import numbers

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

# machine and kernel model
B200_NUM_SMS = 148
KV_TILE_TOKENS = 128               # keys per KV tile of every kernel family
ROWS_PER_WM = 16
SHORT_TILE_ROWS = 16               # row tiles up to this height run on the persistent token-major kernel
WM_CHOICES = (1, 2, 4)
MAX_ROWS_PER_CTA = ROWS_PER_WM * max(WM_CHOICES)
CTAS_PER_SM = {64: 4, 128: 1, 256: 2}   # resident CTAs per SM by head size
SUPPORTED_HEAD_SIZES = tuple(sorted(CTAS_PER_SM))
WINDOWED_HEAD_SIZES = (128,)
ITEMS_PER_SM = 16                  # pieces of work per SM the split bound allows for (the device aims at 8 and rounds)
ALONE_ITEMS_PER_SM = 2             # pieces per SM for a single request
PARTIAL_BYTES_PER_ELEMENT = 4


def _host_int(name: str, value: object, *, at_least: int) -> int:
    """``value`` as an int, refusing bools, tensors and anything else that is not a plain int."""
    if isinstance(value, bool) or not isinstance(value, numbers.Integral) or type(value).__module__ != "builtins":
        raise TypeError(f"{name} must be a host int, got {type(value).__name__}")
    if value < at_least:
        raise ValueError(f"{name} must be >= {at_least}, got {value}")
    return int(value)


def _head_size(D: object) -> int:
    d = _host_int("D", D, at_least=1)
    if d not in CTAS_PER_SM:
        raise ValueError(f"D must be one of {SUPPORTED_HEAD_SIZES}, got {d}")
    return d


def _group_size(G: object) -> int:
    g = _host_int("G", G, at_least=1)
    if g > MAX_ROWS_PER_CTA:
        raise ValueError(f"G must be <= {MAX_ROWS_PER_CTA}, got {g}")
    return g


def _ceil_div(a: int, b: int) -> int:
    return (a + b - 1) // b


def c_target(*, D: int, num_sms: int) -> int:
    """CTAs resident at once: ``num_sms`` x the CTAs of head size ``D`` one SM holds."""
    return CTAS_PER_SM[_head_size(D)] * _host_int("num_sms", num_sms, at_least=1)


def max_tokens_per_tile(G: int) -> int:
    """Query tokens of one request in a 64-row tile."""
    return MAX_ROWS_PER_CTA // _group_size(G)


def wm_for_rows(rows: int) -> int:
    """The smallest ``wm`` whose ``16 * wm`` rows hold ``rows``."""
    need = _host_int("rows", rows, at_least=1)
    fitting = [wm for wm in WM_CHOICES if ROWS_PER_WM * wm >= need]
    if not fitting:
        raise ValueError(f"{need} rows exceed one {MAX_ROWS_PER_CTA}-row tile")
    return fitting[0]


def split_tile_range(*, split: int, num_splits: int, num_tiles: int) -> tuple[int, int]:
    """KV tiles of piece ``split`` when ``num_tiles`` tiles are cut into ``num_splits`` pieces.

    The device's rule (csrc/sched.cuh ``split_tile_span``): piece s is
    ``[s * n // S, (s + 1) * n // S)`` - whole tiles, disjoint, covering, sizes within one.
    """
    pieces = _host_int("num_splits", num_splits, at_least=1)
    which = _host_int("split", split, at_least=0)
    tiles = _host_int("num_tiles", num_tiles, at_least=0)
    if which >= pieces:
        raise ValueError(f"split {which} out of range for num_splits={pieces}")
    return which * tiles // pieces, (which + 1) * tiles // pieces


def s_alone(*, Hkv: int, D: int, num_sms: int) -> int:
    """Pieces a lone row tile per KV head is cut into: every SM gets two of them."""
    heads = _host_int("Hkv", Hkv, at_least=1)
    return max(1, _ceil_div(ALONE_ITEMS_PER_SM * c_target(D=D, num_sms=num_sms), heads))


def _split_bound(unsplit_items: int, *, Hkv: int, D: int, num_sms: int) -> int:
    wanted = _ceil_div(ITEMS_PER_SM * c_target(D=D, num_sms=num_sms), unsplit_items)
    return max(1, min(wanted, s_alone(Hkv=Hkv, D=D, num_sms=num_sms)))


@dataclasses.dataclass(frozen=True)
class LaunchPlan:
    """The host's part of one op call: ``wm`` and ``num_splits`` go to the op as they are."""

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
        return self.Hkv * self.G

    @property
    def rows_per_cta(self) -> int:
        return self.G * self.bq

    @property
    def grid(self) -> tuple[int, int, int]:
        return self.q_tiles_upper, self.Hkv, self.num_splits

    def _partial_splits(self) -> int:
        return 0 if self.num_splits == 1 else self.num_splits

    @property
    def ws_token_splits_used(self) -> int:
        return self._partial_splits() * self.num_tokens

    @property
    def ws_o_shape(self) -> tuple[int, int, int, int]:
        return self._partial_splits(), self.num_tokens, self.Hq, self.D

    @property
    def ws_lse_shape(self) -> tuple[int, int, int]:
        return self._partial_splits(), self.num_tokens, self.Hq


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
    """Plan one op call from the padded batch descriptor of its slice of the batch."""
    tokens = _host_int("num_tokens", num_tokens, at_least=1)
    requests = _host_int("num_reqs", num_reqs, at_least=1)
    longest = _host_int("max_query_len", max_query_len, at_least=1)
    group = _group_size(G)
    heads = _host_int("Hkv", Hkv, at_least=1)
    head_size = _head_size(D)
    sms = _host_int("num_sms", num_sms, at_least=1)
    reserved = _host_int("ws_token_splits", ws_token_splits, at_least=0)
    win = _host_int("window", window, at_least=0)
    if type(is_prefill) is not bool:
        raise TypeError(f"is_prefill must be a bool, got {type(is_prefill).__name__}")
    if longest > tokens:
        raise ValueError(f"max_query_len={longest} > num_tokens={tokens}")
    if tokens > requests * longest:
        raise ValueError(f"num_tokens={tokens} cannot come from {requests} requests of at most {longest} tokens")

    tile_tokens = max_tokens_per_tile(group)
    if is_prefill:
        # Chunks of any length: full 64-row tiles over all tokens.  The bound on the pieces
        # counts REQUESTS, not row tiles: a prefill launch may hold long decode requests of
        # very different lengths (a mixed batch in one launch), which only balance when they
        # may be cut.  The kernels cut on the device and leave the prefill chunks whole, and
        # the bound only matters to a caller that reserved S * T token-splits for such launches.
        wm = max(WM_CHOICES)
        row_tiles = _ceil_div(requests, 2)
    else:
        # every request may be as long as the longest: the fewest tiles that hold it,
        # then the lowest tile that holds its share
        tiles_per_request = _ceil_div(longest, tile_tokens)
        wm = wm_for_rows(group * _ceil_div(longest, tiles_per_request))
        row_tiles = requests * tiles_per_request
    bq = (ROWS_PER_WM * wm) // group

    pieces = _split_bound(heads * row_tiles, Hkv=heads, D=head_size, num_sms=sms)
    pieces = min(pieces, reserved // tokens)   # S > 1 only if S * T fits the reservation
    if win:
        # a row tile sees at most win + longest - 1 keys; at the worst alignment they touch
        touched = _ceil_div(win + longest - 2, KV_TILE_TOKENS) + 1
        pieces = min(pieces, touched)
        if ROWS_PER_WM * wm > SHORT_TILE_ROWS:
            pieces = min(pieces, _ceil_div(sms, heads * row_tiles))
    return LaunchPlan(wm=wm, bq=bq, q_tiles_upper=tokens // bq + requests, num_splits=max(1, pieces),
                      num_tokens=tokens, G=group, Hkv=heads, D=head_size, is_prefill=is_prefill)


def workspace_token_splits(*, max_num_seqs: int, q_dec_max: int, Hkv: int, D: int, num_sms: int) -> int:
    """The reservation ``W_ts`` under which no decode-like plan of this module is clamped.

    A launch of ``r <= max_num_seqs`` requests of up to ``q_dec_max`` tokens asks for
    ``S(r) * T`` token-splits with ``T <= r * q_dec_max``; the bound below takes the worst
    ``r``, with the fewest row tiles such a launch can have (one per request).
    """
    most = _host_int("max_num_seqs", max_num_seqs, at_least=1)
    longest = _host_int("q_dec_max", q_dec_max, at_least=1)
    heads = _host_int("Hkv", Hkv, at_least=1)
    return max(_split_bound(heads * r, Hkv=heads, D=D, num_sms=num_sms) * r * longest for r in range(1, most + 1))


def workspace_shapes(*, ws_token_splits: int, Hq: int, D: int) -> tuple[tuple[int, int, int], tuple[int, int]]:
    """Shapes of the two fp32 buffers to reserve: partial outputs and their log2-sum-exp."""
    rows = _host_int("ws_token_splits", ws_token_splits, at_least=0)
    heads = _host_int("Hq", Hq, at_least=1)
    return (rows, heads, _head_size(D)), (rows, heads)


def workspace_bytes(*, ws_token_splits: int, Hq: int, D: int) -> int:
    """Bytes of both buffers together: ``W_ts * Hq * (D + 1) * 4``."""
    (rows, heads, head_size), _ = workspace_shapes(ws_token_splits=ws_token_splits, Hq=Hq, D=D)
    return rows * heads * (head_size + 1) * PARTIAL_BYTES_PER_ELEMENT
