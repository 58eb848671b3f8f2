"""Out-of-bounds WRITE detection with guard zones (a stand-in for a memory checker where none
can run).  Every buffer a kernel writes -- outputs, side outputs, and the scratch
whose size the library itself reports -- is carved out of the middle of a poisoned arena with 16 KiB of canaries on
each side, at EXACTLY the size the API asks for; after the kernel the canaries must be intact.  Run over the hand-rolled
pipelines: the streaming decode kernels (mbarrier rings, chunk partials, in-kernel row merge), the
split-KV grid kernel + merge kernels, the beam-group kernel, the tcgen05 GEMM (direct, split-K scratch, fused
dynamic-quantisation epilogue), the tcgen05 prefill, the row append and the exchange.  Results are also checked against
the oracle, so a kernel cannot pass by writing nothing."""
import numpy as np
import pytest
import torch

from synth import make_case, oracle_attention, to_device_cache

pytestmark = pytest.mark.gpu
GUARD = 16384
POISON = 0xA5


class Arena:
    """Carves exact-size buffers with guard zones out of one poisoned uint8 allocation."""

    def __init__(self, nbytes):
        self.buf = torch.full((nbytes,), POISON, dtype=torch.uint8, device="cuda")
        self.off = 0
        self.guards = []

    def take(self, nbytes, dtype=torch.uint8, shape=None, align=256):
        self.off = (self.off + align - 1) // align * align
        g0 = (self.off, self.off + GUARD)
        start = g0[1]
        start = (start + align - 1) // align * align
        end = start + nbytes
        g1 = (end, end + GUARD)
        self.guards += [(g0[0], start), g1]
        self.off = g1[1]
        assert self.off <= self.buf.numel(), "arena too small"
        t = self.buf[start:end].view(dtype)
        return t.view(shape) if shape is not None else t

    def check(self, what):
        torch.cuda.synchronize()
        for a, b in self.guards:
            bad = (self.buf[a:b] != POISON).nonzero()
            assert bad.numel() == 0, f"{what}: guard zone [{a}, {b}) overwritten at byte {a + int(bad[0])}"


@pytest.fixture(scope="module")
def ld(oracle):
    import llm_decoder
    return llm_decoder


@pytest.mark.parametrize("kv", ["f16", "i8", "f32"])
@pytest.mark.parametrize("overlap", [False, True])
@pytest.mark.parametrize("shape", [dict(B=3, H=5, D=128, T=1000, ragged=True), dict(B=1, H=4, D=128, T=16384),
                                   dict(B=2, H=3, D=64, T=333, unmapped_frac=0.05)])
def test_decode_outputs_and_workspace_stay_in_bounds(ld, oracle, kv, overlap, shape):
    from llm_decoder import _cabi
    lib = _cabi.lib()
    case = make_case(seed=81, kv=kv, **shape)
    kvc = to_device_cache(case)
    B, H, D = case["q"].shape
    pt = kvc.page_table_
    need = lib.pa_decode_workspace_bytes(B, H, D, pt.num_tiles_, kvc.tile_size_)
    ar = Arena(need + B * H * (D + 1) * 4 + 8 * GUARD + 4096)
    out = ar.take(B * H * D * 4, torch.float32, (B, H, D))
    lse = ar.take(B * H * 4, torch.float32, (B, H))
    ws = ar.take(need)
    q = torch.from_numpy(case["q"]).cuda()
    ctx = None if case["ctx_lens"] is None else torch.from_numpy(case["ctx_lens"]).cuda()
    name = {"f16": "pa_paged_decode_f16", "i8": "pa_paged_decode_i8", "f32": "pa_paged_decode_f32"}[kv] + ("_overlap" if overlap else "")
    pools = (kvc.key_buffer_.data_ptr(), kvc.value_buffer_.data_ptr())
    if kv == "i8":
        pools += (kvc.k_scales_.data_ptr(), kvc.v_scales_.data_ptr())
    for _ in range(2):
        _cabi.check(getattr(lib, name)(q.data_ptr(), out.data_ptr(), *pools, pt.device_data().data_ptr(), pt.num_beams_, H,
                                       pt.num_tiles_, kvc.total_pages_, None, _cabi.ptr(ctx), B, case["T"], D, kvc.tile_size_,
                                       case["temperature"], None, lse.data_ptr(), ws.data_ptr(), need, None), name)
        ar.check(name)
    np.testing.assert_allclose(out.cpu().numpy(), oracle_attention(case), rtol=2e-3, atol=1e-3)


def test_group_and_partial_kernels_stay_in_bounds(ld, oracle):
    from llm_decoder import _cabi
    lib = _cabi.lib()
    case = make_case(B=8, H=3, D=128, T=640, seed=82, beam_width=4, shared_prefix=384)
    kvc = to_device_cache(case)
    B, H, D = case["q"].shape
    pt = kvc.page_table_
    need = lib.pa_decode_workspace_bytes(B, H, D, pt.num_tiles_, kvc.tile_size_)
    ar = Arena(2 * need + 4 * B * H * (D + 2) * 4 + 16 * GUARD + 8192)
    out = ar.take(B * H * D * 4, torch.float32, (B, H, D))
    ws = ar.take(need)
    q = torch.from_numpy(case["q"]).cuda()
    beams = torch.from_numpy(case["beam_ids"]).cuda()
    _cabi.check(lib.pa_paged_decode_f16_group(q.data_ptr(), out.data_ptr(), kvc.key_buffer_.data_ptr(), kvc.value_buffer_.data_ptr(),
                                              pt.device_data().data_ptr(), pt.num_beams_, H, pt.num_tiles_, kvc.total_pages_,
                                              beams.data_ptr(), None, B, case["T"], D, kvc.tile_size_, case["temperature"], None, 4,
                                              None, ws.data_ptr(), need, None), "group")
    ar.check("pa_paged_decode_f16_group")
    np.testing.assert_allclose(out.cpu().numpy(), oracle_attention(case), rtol=2e-3, atol=1e-3)
    pm = ar.take(B * H * 4, torch.float32)
    pl = ar.take(B * H * 4, torch.float32)
    po = ar.take(B * H * D * 4, torch.float32)
    ws2 = ar.take(need)
    _cabi.check(lib.pa_paged_decode_f16_partial(q.data_ptr(), pm.data_ptr(), pl.data_ptr(), po.data_ptr(), kvc.key_buffer_.data_ptr(),
                                                kvc.value_buffer_.data_ptr(), pt.device_data().data_ptr(), pt.num_beams_, H,
                                                pt.num_tiles_, kvc.total_pages_, beams.data_ptr(), None, B, case["T"], D,
                                                kvc.tile_size_, case["temperature"], None, ws2.data_ptr(), need, None), "partial")
    ar.check("pa_paged_decode_f16_partial")
    got = (po.view(B * H, D) / (pl.unsqueeze(-1) + 1e-6)).cpu().numpy().reshape(B, H, D)
    np.testing.assert_allclose(got, oracle_attention(case), rtol=2e-3, atol=1e-3)


@pytest.mark.parametrize("shape", [(256, 512, 256), (300, 272, 128), (8, 768, 3072), (64, 3072, 768), (256, 4096, 1024)])
def test_gemm_outputs_and_scratch_stay_in_bounds(ld, oracle, shape):
    from llm_decoder import _cabi
    lib = _cabi.lib()
    M, N, K = shape
    rng = np.random.default_rng(83)
    A = torch.from_numpy(rng.integers(-127, 128, (1, M, K), dtype=np.int8)).cuda()
    Bm = torch.from_numpy(rng.integers(-127, 128, (1, K, N), dtype=np.int8)).cuda()
    bias = torch.from_numpy(rng.standard_normal(N).astype(np.float32)).cuda()
    qs = torch.from_numpy(rng.uniform(5, 60, M).astype(np.float32)).cuda()
    need = lib.pa_gemm_i8_workspace_bytes(1, M, N, K)
    dqn = lib.pa_gemm_i8_dynquant_workspace_bytes(1, M, N)
    ar = Arena(M * N * (1 + 4 + 4 + 1) + need + dqn + M * 4 + 16 * GUARD + 8192)
    c8 = ar.take(M * N, torch.int8, (1, M, N))
    c32 = ar.take(M * N * 4, torch.int32, (1, M, N))
    cf = ar.take(M * N * 4, torch.float32, (1, M, N))
    ws = ar.take(max(need, 16))
    _cabi.check(lib.pa_gemm_i8(A.data_ptr(), Bm.data_ptr(), c8.data_ptr(), c32.data_ptr(), 1, M, N, K, 1 / 16, 1 / 16, 8.0,
                               bias.data_ptr(), 1, ws.data_ptr(), need, None), "pa_gemm_i8")
    ar.check("pa_gemm_i8")
    np.testing.assert_array_equal(c32.cpu().numpy(), oracle.cpu.gemm_s8s8s32(A.cpu().numpy(), Bm.cpu().numpy()))
    _cabi.check(lib.pa_gemm_i8_dequant(A.data_ptr(), Bm.data_ptr(), cf.data_ptr(), 1, M, N, K, qs.data_ptr(), 0.01, bias.data_ptr(), 0,
                                       ws.data_ptr(), need, None), "pa_gemm_i8_dequant")
    ar.check("pa_gemm_i8_dequant")
    if M > 128:
        q8 = ar.take(M * N, torch.int8, (1, M, N))
        sc = ar.take(M * 4, torch.float32)
        dws = ar.take(dqn)
        dws.zero_()
        st = lib.pa_gemm_i8_dynquant(A.data_ptr(), Bm.data_ptr(), q8.data_ptr(), sc.data_ptr(), 1, M, N, K, qs.data_ptr(), 0.01,
                                     bias.data_ptr(), 1, dws.data_ptr(), dqn, None)
        if st != -2:
            _cabi.check(st, "pa_gemm_i8_dynquant")
            ar.check("pa_gemm_i8_dynquant")
            assert (dws[:16] == 0).all()    # the barrier words are left zero


def test_append_touches_only_its_rows(ld, oracle):
    """pa_kv_append_*: exactly the addressed (page, row) slots change; every other byte of the pools and scales stays."""
    for kv in ("f16", "i8", "f32"):
        case = make_case(B=4, H=3, D=128, T=96, seed=84, kv=kv, unmapped_frac=0.1)
        kvc = to_device_cache(case)
        k0, v0 = kvc.key_buffer_.clone(), kvc.value_buffer_.clone()
        rng = np.random.default_rng(84)
        nk = torch.from_numpy(rng.standard_normal((4, 3, 128)).astype(np.float32)).cuda()
        nv = torch.from_numpy(rng.standard_normal((4, 3, 128)).astype(np.float32)).cuda()
        pos = torch.tensor([0, 17, 95, 200], dtype=torch.int32, device="cuda")   # 200: out of range -> no write
        kvc.append(nk, nv, pos)
        torch.cuda.synchronize()
        tb = case["table"]
        touched = torch.zeros(kvc.key_buffer_.shape[:2], dtype=torch.bool)
        for r, p in enumerate([0, 17, 95]):
            for h in range(3):
                pg = tb[r, h, p // 16]
                if 0 <= pg < case["total_pages"]:
                    touched[pg, p % 16] = True
        same_k = (kvc.key_buffer_ == k0).all(dim=2).cpu()
        same_v = (kvc.value_buffer_ == v0).all(dim=2).cpu()
        assert same_k[~touched].all() and same_v[~touched].all(), kv


def test_prefill_output_stays_in_bounds(ld, oracle):
    from llm_decoder import _cabi
    lib = _cabi.lib()
    for kv in ("f16", "i8"):
        case = make_case(B=2, H=2, D=128, T=320, seed=85, kv=kv)
        kvc = to_device_cache(case)
        B, H, D, Tq = 2, 2, 128, 300
        pt = kvc.page_table_
        ar = Arena(B * H * Tq * D * 4 + 4 * GUARD + 4096)
        out = ar.take(B * H * Tq * D * 4, torch.float32, (B, H, Tq, D))
        q = torch.randn((B, H, Tq, D), device="cuda")
        pools = (kvc.key_buffer_.data_ptr(), kvc.value_buffer_.data_ptr())
        fn = lib.pa_paged_prefill_f16
        if kv == "i8":
            fn = lib.pa_paged_prefill_i8
            pools += (kvc.k_scales_.data_ptr(), kvc.v_scales_.data_ptr())
        _cabi.check(fn(q.data_ptr(), out.data_ptr(), *pools, pt.device_data().data_ptr(), pt.num_beams_, H, pt.num_tiles_,
                       kvc.total_pages_, None, None, B, Tq, D, kvc.tile_size_, case["temperature"], None, 0, None), "prefill")
        ar.check("pa_paged_prefill_" + kv)
        assert torch.isfinite(out).all()
