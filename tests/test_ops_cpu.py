"""The torch op on the CPU dispatch key: every argument check runs without a GPU, the Python
fake kernel raises the same text, and a valid CPU call refuses to compute."""
import re

import pytest
import torch

from pth_flash_attn_b200 import ops

pytestmark = pytest.mark.skipif(not ops.is_available(), reason="op library not built")


def make_args(T=3, Hq=8, Hkv=2, D=128, NB=4, BS=16, R=2, S=1, dtype=torch.bfloat16):
    C = 2 * (D + 4)
    storage = torch.zeros(NB * BS * Hkv * C, dtype=torch.int8)
    packed = storage.view(NB, BS, Hkv, C)
    k_cache, v_cache = packed[..., :D], packed[..., D + 4: 2 * D + 4]
    f32 = storage.view(torch.float32).view(NB, BS, Hkv, C // 4)
    k_scale, v_scale = f32[..., D // 4], f32[..., C // 4 - 1]
    a = dict(
        out=torch.zeros(T, Hq, D, dtype=dtype), q=torch.zeros(T, Hq, D, dtype=dtype), k_cache=k_cache,
        v_cache=v_cache, k_scale=k_scale, v_scale=v_scale,
        block_table=torch.zeros(R, 4, dtype=torch.int32), seq_lens=torch.ones(R, dtype=torch.int32),
        query_start_loc=torch.zeros(R + 1, dtype=torch.int32), max_query_len=T, wm=1, num_splits=S,
        softmax_scale=D ** -0.5,
        ws_o=torch.zeros(S if S > 1 else 0, T, Hq, D), ws_lse=torch.zeros(S if S > 1 else 0, T, Hq),
        window=0, causal=True)
    return a


def call(a):
    ops.pth_flash_attn_fwd(**a)


def message_of(fn, a):
    with pytest.raises(RuntimeError) as e:
        fn(a)
    text = str(e.value)
    m = re.search(r"pth_flash_attn_fwd: .*", text)
    return m.group(0).split("\n")[0] if m else text


def test_schema_is_frozen():
    schema = torch.ops.pth_flash_attn.pth_flash_attn_fwd.default._schema
    want = ("pth_flash_attn::" + ops.OP_SCHEMA).replace("Tensor! ", "Tensor(a!) ")
    norm = lambda s: re.sub(r"Tensor\([^)]*![^)]*\)", "Tensor!", str(s)).replace(" ", "")  # noqa: E731
    assert norm(schema) == norm("pth_flash_attn::" + ops.OP_SCHEMA)
    assert want  # the textual schema is part of the documented integration contract


def test_valid_cpu_call_refuses_to_compute():
    assert "computes on CUDA tensors only" in message_of(call, make_args())
    assert "computes on CUDA tensors only" in message_of(call, make_args(S=3))


def test_legacy_15_argument_call_resolves():
    a = make_args()
    a.pop("window"), a.pop("causal")
    with pytest.raises(RuntimeError, match="computes on CUDA tensors only"):
        torch.ops.pth_flash_attn.pth_flash_attn_fwd(*a.values())


def _bad_cases():
    def case(name, needle, **make_kw):
        def deco(fn):
            cases.append((name, needle, make_kw, fn))
            return fn
        return deco

    cases = []
    case("q dtype", "q must be bfloat16 or float16")(lambda a: a.update(q=a["q"].float()))
    case("q rank", "q must be 3-D")(lambda a: a.update(q=a["q"][0]))
    case("D=96", "head size D = q.size(2) must be 64, 128 or 256", D=96)(lambda a: None)
    case("q inner stride", "q must have stride 1")(lambda a: a.update(q=torch.zeros(3, 8, 256, dtype=torch.bfloat16)[..., ::2]))
    case("out dtype", "out (same dtype as q) must be bfloat16")(lambda a: a.update(out=a["out"].half()))
    case("out shape", "out.size(0) must equal T")(lambda a: a.update(out=torch.zeros(4, 8, 128, dtype=torch.bfloat16)))
    case("cache dtype", "k_cache must be int8")(lambda a: a.update(k_cache=a["k_cache"].to(torch.int32)))
    case("cache rank", "v_cache must be 4-D")(lambda a: a.update(v_cache=a["v_cache"][0]))
    case("cache D", "k_cache.size(3) must equal D")(lambda a: a.update(k_cache=a["k_cache"][..., :64]))
    case("cache BS", "v_cache.size(1) must equal BS")(lambda a: a.update(v_cache=a["v_cache"][:, :8]))
    case("scale dtype", "k_scale must be float32")(lambda a: a.update(k_scale=a["k_scale"].double()))
    case("scale shape", "v_scale.size(2) must equal Hkv")(lambda a: a.update(v_scale=a["v_scale"][..., :1]))
    case("Hq % Hkv", "must be a positive multiple of Hkv", Hq=7)(lambda a: None)
    case("wm=3", "wm must be 1, 2 or 4")(lambda a: a.update(wm=3))
    case("G > 16 wm", "must be <= 16*wm", Hq=64)(lambda a: None)
    case("G > 64", "exceeds the supported maximum", Hq=130, Hkv=1)(lambda a: a.update(wm=4))
    case("bt dtype", "block_table must be int32")(lambda a: a.update(block_table=a["block_table"].long()))
    case("lens rank", "seq_lens must be 1-D")(lambda a: a.update(seq_lens=a["seq_lens"][None]))
    case("qsl length", "query_start_loc.size(0) must equal num_reqs + 1")(lambda a: a.update(query_start_loc=torch.zeros(5, dtype=torch.int32)))
    case("bt rows", "rows, fewer than num_reqs")(lambda a: a.update(block_table=a["block_table"][:1]))
    case("max_query_len", "max_query_len must be in [0, T")(lambda a: a.update(max_query_len=4))
    case("num_splits 0", "num_splits must be >= 1")(lambda a: a.update(num_splits=0))
    case("scale nan", "softmax_scale must be finite and > 0")(lambda a: a.update(softmax_scale=float("nan")))
    case("scale 0", "softmax_scale must be finite and > 0")(lambda a: a.update(softmax_scale=0.0))
    case("window < 0", "window must be >= 0")(lambda a: a.update(window=-1))
    case("window off D128", "need head size D = 128", D=64)(lambda a: a.update(window=8))
    case("non-causal off D128", "need head size D = 128", D=256)(lambda a: a.update(causal=False))
    case("S=2 no workspace", "ws_o must be 4-D")(lambda a: a.update(num_splits=2, ws_o=torch.zeros(0)))
    case("ws few splits", "ws_o must have size(0) >= num_splits", S=2)(lambda a: a.update(num_splits=3))
    case("ws few tokens", "ws_lse must have size(0) >= num_splits", S=2)(lambda a: a.update(ws_lse=torch.zeros(2, 2, 8)))
    case("ws Hq", "ws_o.size(2) must equal Hq", S=2)(lambda a: a.update(ws_o=torch.zeros(2, 3, 4, 128)))
    case("ws dtype", "ws_o must be float32", S=2)(lambda a: a.update(ws_o=a["ws_o"].half()))
    return cases


@pytest.mark.parametrize("name,needle,make_kw,mutate", _bad_cases(), ids=[c[0] for c in _bad_cases()])
def test_invalid_arguments(name, needle, make_kw, mutate):
    a = make_args(**make_kw)
    mutate(a)
    cpp = message_of(call, a)
    assert needle in cpp, cpp
    # the fake kernel raises the same text
    fake = message_of(lambda x: ops.pth_flash_attn_fwd_fake(**x), a)
    assert fake == cpp


def test_address_checks_are_cpp_only():
    a = make_args()
    store = torch.zeros(3 * 8 * 128 + 8, dtype=torch.bfloat16)
    a["q"] = store[4:4 + 3 * 8 * 128].view(3, 8, 128)  # 8-byte offset
    assert "q data pointer must be 16-byte aligned" in message_of(call, a)
    a = make_args()
    odd = torch.zeros(a["k_cache"].numel() * 3, dtype=torch.int8)
    a["k_cache"] = torch.as_strided(odd, a["k_cache"].shape, a["k_cache"].stride(), 1)
    assert "k_cache data pointer must be 4-byte aligned" in message_of(call, a)
    a = make_args()
    a["v_scale"] = torch.as_strided(torch.zeros(1 << 16), (4, 16, 2), (16 * 2 * 66 + 1, 2 * 66, 66))
    assert "v_scale byte stride of dim 0" not in message_of(call, a)  # fp32 strides are 4-byte multiples


def test_fake_kernel_returns_none_and_touches_nothing():
    a = make_args()
    a["out"].fill_(3.0)
    assert ops.pth_flash_attn_fwd_fake(**a) is None
    assert (a["out"] == 3.0).all()


def test_lse_variant_checks_its_output():
    a = make_args()
    with pytest.raises(RuntimeError, match="lse must be float32"):
        ops.pth_flash_attn_fwd_lse(a["out"], torch.zeros(3, 8, dtype=torch.float16), *list(a.values())[1:])
    with pytest.raises(RuntimeError, match="computes on CUDA tensors only"):
        ops.pth_flash_attn_fwd_lse(a["out"], torch.zeros(3, 8), *list(a.values())[1:])


def test_module_makes_no_cuda_call():
    import inspect

    src = inspect.getsource(ops)
    assert "torch.cuda" not in src.replace("``torch.cuda``", "")
