"""Full-size parity: the 7B prefill and decode shapes and the MoE block at its real dimensions.

The operands are generated on the GPU from a seed (the exporter's own kernel quantises the weights,
and its bytes equal the oracle's bit for bit, tests/test_gpu_export.py), the CUDA path runs on the whole
problem, and the CPU oracle recomputes a SAMPLE of the output -- a set of rows and a set of columns
(tokens, for the MoE block) -- from the same operands with exact accumulation.  Tolerances as in
tests/test_gpu_linear.py (T1; 3 x T1 for the three-rounding expert FFN).
"""
import importlib

import numpy as np
import pytest
import torch

from oracle import fp8_oracle as O
from helpers import assert_parity, from_bf16, kernels

pytestmark = pytest.mark.gpu

KNOBS = ("umma_pair", "umma_bn", "umma_splits", "swap_min_m", "w8a16_swap_min_m", "fuse_quant")


@pytest.fixture(autouse=True)
def _clean():
    yield
    Kn = kernels()
    for knob in KNOBS:
        Kn.set_tuning(knob, -1)
    torch.cuda.synchronize()
    assert Kn.read_status(torch.device("cuda", 0)) == 0
    torch.cuda.empty_cache()


def quantize_on_gpu(w):
    """[N, K] float weights on the device -> (codes [N, K] uint8, scale [N]) by the exporter's kernel."""
    exp = importlib.import_module("nano-vllm-moe_b200.quantization.export")
    return exp.quantize_weight(w)


def big_case(seed, m, k, n):
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn((m, k), generator=g, device="cuda", dtype=torch.float32).to(torch.bfloat16)
    w = torch.randn((n, k), generator=g, device="cuda", dtype=torch.float32) * 0.02
    q, s = quantize_on_gpu(w)
    del w
    bias = (torch.randn((n,), generator=g, device="cuda") * 0.01).to(torch.bfloat16)
    calib = torch.randn((1024, k), generator=g, device="cuda").to(torch.bfloat16)
    in_scale = (calib.float().abs().amax() / 448.0).to(torch.float32).reshape(())
    Kn = kernels()
    return {"x": x, "q": q.view(torch.uint8), "w_scale": s, "bias": bias, "input_scale": in_scale,
            "w_nk": Kn.pack_weight_nk(q.view(torch.uint8))}


def sample(size, count, rng, edges=True):
    """`count` sorted indices of range(size), always holding the first and the last few (tile tails)."""
    if size <= count:
        return np.arange(size)
    pick = set(rng.choice(size, count, replace=False).tolist())
    if edges:
        pick |= {0, 1, size - 1, size - 2, size // 2}
    return np.array(sorted(pick))


def check_sampled(scheme, d, y, rows, cols, what, ulps=1.0):
    x = from_bf16(d["x"][torch.from_numpy(rows).cuda()])
    ct = torch.from_numpy(cols).cuda()
    wq = d["q"][ct].cpu().numpy()
    ws = d["w_scale"][ct].cpu().numpy()
    b = from_bf16(d["bias"][ct])
    if scheme == "fp8_w8a16":
        ref = O.linear_w8a16(x, wq, ws, b)
    else:
        ref = O.linear_w8a8(x, wq, ws, np.float32(d["input_scale"].item()), b)
    got = from_bf16(y[torch.from_numpy(rows).cuda()][:, ct])
    assert_parity(got, ref, what, ulps=ulps)


def run(scheme, d):
    Kn = kernels()
    if scheme == "fp8_w8a16":
        return Kn.launch_w8a16_gemm(d["x"], d["w_nk"], d["w_scale"], d["bias"])
    return Kn.launch_w8a8_gemm(d["x"], d["w_nk"], d["input_scale"], d["w_scale"], d["bias"])


# (M, K, N, forced umma_pair or None, substring expected in the variant name)
PREFILL = [
    (4096, 18944, 3584, None, "+tail"),            # persistent launch + cluster split-K tail launch
    (2048, 8192, 2560, None, "+tail"),             # the same route on a small problem
    (16384, 18944, 3584, None, "+tail"),
    (16384, 3584, 3584, None, "+half"),
    (32640, 3584, 4608, 0, "umma_w8a8"),           # ragged M (32640 = 255 x 128), one-CTA kernel
    (32640, 3584, 4608, 1, "umma_pair"),           # ragged M on CTA pairs: the last pair has one live CTA row block
    (4096, 3584, 37888, None, "umma_pair"),        # gate_up on CTA pairs (148 column tiles)
    (32640, 18944, 3584, None, "umma_pair"),
    (16384, 3584, 576, None, "umma_w8a8_128x256"), # qkv and gate_up column shards of 8 ranks (N = 4.5 and 37 tiles of 128)
    (16384, 3584, 4736, None, "umma_pair"),
    (16384, 2368, 3584, None, "+half"),            # down's K shard of 8 ranks: 18.5 K blocks
]


@pytest.mark.parametrize("m,k,n,pair,expect", PREFILL)
def test_prefill_shapes_sampled(m, k, n, pair, expect):
    Kn = kernels()
    if pair is not None:
        Kn.set_tuning("umma_pair", pair)
    name = Kn.variant_name(1, m, k, n)
    assert expect in name, name
    d = big_case(m + k + n, m, k, n)
    y = run("fp8_w8a8_static", d)              # default: a separate pass quantises the activations
    rng = np.random.default_rng(m + n)
    rows, cols = sample(m, 48, rng), sample(n, 160, rng)
    check_sampled("fp8_w8a8_static", d, y, rows, cols, f"{name} {m}x{k}x{n}")
    # every row block and column block is written: no element keeps the fill value
    assert torch.isfinite(y.float()).all()
    assert torch.equal(y, run("fp8_w8a8_static", d))
    Kn.set_tuning("fuse_quant", 1)             # rows past the first round of tiles quantised inside the GEMM: same bits
    assert torch.equal(y, run("fp8_w8a8_static", d))


@pytest.mark.parametrize("first_rows", [128, 640])
@pytest.mark.parametrize("m,k,n", [(2304, 256, 512), (1500, 448, 264), (4096, 2048, 1024), (300, 144, 72)])
def test_in_kernel_quantiser_small_shapes_exact(m, k, n, first_rows):
    """Only the first `first_rows` rows are quantised ahead of the GEMM, so its first tiles really wait for the
    kernel's own quantiser warps (ragged last row block, K and N tails), on the one-CTA kernel and on CTA pairs:
    whole output against the oracle and against the separate pass."""
    from helpers import oracle_linear, upload_case
    Kn = kernels()
    c = O.make_case(31 + m, m, k, n, calib_rows=256)
    d = upload_case(c)
    ref = oracle_linear("fp8_w8a8_static", c)
    for pair in (0, 1):
        Kn.set_tuning("umma_pair", pair)
        Kn.set_tuning("fuse_quant", first_rows)
        y = Kn.launch_w8a8_gemm(d["x"], d["w_nk"], d["input_scale"], d["w_scale"], d["bias"])
        assert_parity(from_bf16(y), ref, f"in-kernel quantiser pair={pair} {m}x{k}x{n}")
        Kn.set_tuning("fuse_quant", 0)
        assert torch.equal(y, Kn.launch_w8a8_gemm(d["x"], d["w_nk"], d["input_scale"], d["w_scale"], d["bias"]))


LAYERS = {"qkv": (3584, 4608), "o_proj": (3584, 3584), "gate_up": (3584, 37888), "down": (18944, 3584)}


@pytest.mark.parametrize("scheme", ["fp8_w8a8_static", "fp8_w8a16"])
@pytest.mark.parametrize("layer", list(LAYERS))
def test_decode_sweep_all_layers(scheme, layer):
    """The 7B decode grid: M in {1, 4, 16, 64} on each of the four layer shapes, both schemes, default routing."""
    k, n = LAYERS[layer]
    d = big_case(k + n, 64, k, n)
    rng = np.random.default_rng(n)
    cols = sample(n, 192, rng)
    full_x = d["x"]
    for m in (1, 4, 16, 64):
        d["x"] = full_x[:m].contiguous()
        y = run(scheme, d)
        name = kernels().variant_name(0 if scheme == "fp8_w8a16" else 1, m, k, n)
        check_sampled(scheme, d, y, np.arange(m), cols, f"{scheme} {layer} M={m} [{name}]")
        assert torch.isfinite(y.float()).all()


@pytest.mark.parametrize("T", [1, 1024, 4096])
def test_moe_block_real_dimensions_sampled_tokens(T):
    """Hidden 2048, 60 experts, intermediate 1408, top-4: the whole step on the GPU, a sample of tokens on the CPU."""
    moe = importlib.import_module("nano-vllm-moe_b200.executor.moe")
    H, E, I, K = 2048, 60, 1408, 4
    g = torch.Generator(device="cuda").manual_seed(90 + T)
    x = torch.randn((T, H), generator=g, device="cuda").to(torch.bfloat16)
    logits = torch.randn((T, E), generator=g, device="cuda")
    q13, s13, q2, s2 = [], [], [], []
    for e in range(E):
        q, s = quantize_on_gpu(torch.randn((2 * I, H), generator=g, device="cuda") * 0.02); q13.append(q.view(torch.uint8)); s13.append(s)
        q, s = quantize_on_gpu(torch.randn((H, I), generator=g, device="cuda") * 0.02); q2.append(q.view(torch.uint8)); s2.append(s)
    q13, s13, q2, s2 = torch.stack(q13), torch.stack(s13), torch.stack(q2), torch.stack(s2)
    in13 = (torch.randn((1024, H), generator=g, device="cuda").to(torch.bfloat16).float().abs().amax() / 448.0).reshape(())
    in2 = torch.tensor(4.0 / 448.0, device="cuda")
    wts = moe.Fp8ExpertWeights.from_checkpoint_layout(q13, s13, in13, q2, s2, in2)
    cfg = moe.make_moe_parallel_config(tp_group=None, ep_group=None, global_num_experts=E, intermediate_size=I)
    kern = moe.MoEKernel(prepare_finalize=moe.NoEPPrepareFinalize(cfg), experts=moe.Fp8Experts(), parallel_config=cfg)
    w, ids = moe.SoftmaxTopKRouter(K, False).select_experts(None, logits)
    y = kern(x, w, ids, wts, model_dtype=torch.bfloat16)
    assert torch.equal(y, kern(x, w, ids, wts, model_dtype=torch.bfloat16))
    tok = sample(T, 24, np.random.default_rng(T))
    tt = torch.from_numpy(tok).cuda()
    w_ref, ids_ref = O.softmax_topk(logits[tt].cpu().numpy(), K, False)
    np.testing.assert_array_equal(ids[tt].cpu().numpy(), ids_ref)
    ref = O.moe_experts_w8a8(from_bf16(x[tt]), ids_ref, w_ref, q13.cpu().numpy(), s13.cpu().numpy(), np.float32(in13.item()),
                             q2.cpu().numpy(), s2.cpu().numpy(), np.float32(in2.item()))
    assert_parity(from_bf16(y[tt]), ref, f"moe block T={T}", ulps=3.0, min_cos=0.9999)


def test_row_grouping_matches_reference_alignment(golden):
    """fp8lin_moe_align on the routing the reference's moe_align_block_size was recorded on: the same rows
    per expert (order inside an expert is free), every kept row exactly once, chunks of one expert each."""
    pkg = importlib.import_module("nano-vllm-moe_b200")
    lib = pkg._lib.load()
    g = golden("moe")
    ids_np = g["topk_ids_ren0"].reshape(-1).astype(np.int32)
    E, rows = 12, ids_np.size
    ref_rows, ref_experts = g["align_sorted_weight_idx"], g["align_expert_ids"]
    want = {e: set() for e in range(E)}
    for b, e in enumerate(ref_experts):
        blk = ref_rows[b * 8:(b + 1) * 8]
        want[int(e)] |= set(int(r) for r in blk[blk < rows])
    ids = torch.from_numpy(ids_np).cuda()
    for chunk_rows in (16, 32, 64, 128):
        offs = torch.full((E + 1,), -1, dtype=torch.int32, device="cuda")
        srt = torch.full((rows,), -1, dtype=torch.int32, device="cuda")
        chunks = torch.full((E + rows // 16 + 2, 4), -1, dtype=torch.int32, device="cuda")
        meta = torch.full((2,), -1, dtype=torch.int32, device="cuda")
        rc = lib.fp8lin_moe_align(ids.data_ptr(), rows, E, chunk_rows, offs.data_ptr(), srt.data_ptr(), chunks.data_ptr(),
                                  meta.data_ptr(), torch.cuda.current_stream().cuda_stream)
        pkg._lib.raise_for(rc, "fp8lin_moe_align")
        offs, srt, chunks, meta = offs.cpu().numpy(), srt.cpu().numpy(), chunks.cpu().numpy(), meta.cpu().numpy()
        assert meta[1] == rows and offs[0] == 0 and offs[E] == rows
        for e in range(E):
            assert set(srt[offs[e]:offs[e + 1]].tolist()) == want[e], e
        np.testing.assert_array_equal(np.sort(srt), np.arange(rows))
        covered = np.zeros(rows, bool)
        for e, first, cnt, _ in chunks[:meta[0]]:
            assert 0 < cnt <= chunk_rows and offs[e] <= first and first + cnt <= offs[e + 1]
            assert not covered[first:first + cnt].any()
            covered[first:first + cnt] = True
        assert covered.all()
    # ids outside [0, E) belong to another expert-parallel rank: dropped
    mixed = ids.clone(); mixed[::3] = -1; mixed[1::5] = E + 2
    keep = ((mixed >= 0) & (mixed < E)).sum().item()
    offs = torch.zeros((E + 1,), dtype=torch.int32, device="cuda"); srt = torch.zeros((rows,), dtype=torch.int32, device="cuda")
    chunks = torch.zeros((E + rows // 16 + 2, 4), dtype=torch.int32, device="cuda"); meta = torch.zeros((2,), dtype=torch.int32, device="cuda")
    pkg._lib.raise_for(lib.fp8lin_moe_align(mixed.data_ptr(), rows, E, 16, offs.data_ptr(), srt.data_ptr(), chunks.data_ptr(),
                                            meta.data_ptr(), torch.cuda.current_stream().cuda_stream), "fp8lin_moe_align")
    assert meta.cpu().numpy()[1] == keep
    kept = srt.cpu().numpy()[:keep]
    assert ((mixed.cpu().numpy()[kept] >= 0) & (mixed.cpu().numpy()[kept] < E)).all()


@pytest.mark.parametrize("rows,E", [(5000, 60), (16384, 60), (2048, 128), (3000, 7), (4097, 129)])
def test_row_grouping_many_rows(rows, E):
    """Prefill-sized batches: every kept row exactly once, rows of an expert adjacent, chunks inside one expert, and
    the per-expert counts of a numpy bincount."""
    pkg = importlib.import_module("nano-vllm-moe_b200")
    lib = pkg._lib.load()
    rng = np.random.default_rng(rows + E)
    ids_np = rng.integers(-1, E + 1, size=rows).astype(np.int32)            # a few ids outside [0, E): dropped
    valid = (ids_np >= 0) & (ids_np < E)
    ids = torch.from_numpy(ids_np).cuda()
    offs = torch.full((E + 1,), -1, dtype=torch.int32, device="cuda")
    srt = torch.full((rows,), -1, dtype=torch.int32, device="cuda")
    chunks = torch.full((E + rows // 16 + 2, 4), -1, dtype=torch.int32, device="cuda")
    meta = torch.full((2,), -1, dtype=torch.int32, device="cuda")
    pkg._lib.raise_for(lib.fp8lin_moe_align(ids.data_ptr(), rows, E, 128, offs.data_ptr(), srt.data_ptr(), chunks.data_ptr(),
                                            meta.data_ptr(), torch.cuda.current_stream().cuda_stream), "fp8lin_moe_align")
    offs, srt, chunks, meta = offs.cpu().numpy(), srt.cpu().numpy(), chunks.cpu().numpy(), meta.cpu().numpy()
    counts = np.bincount(ids_np[valid], minlength=E)
    np.testing.assert_array_equal(np.diff(offs), counts)
    kept = srt[:meta[1]]
    assert meta[1] == valid.sum()
    np.testing.assert_array_equal(np.sort(kept), np.flatnonzero(valid))
    np.testing.assert_array_equal(ids_np[kept], np.repeat(np.arange(E), counts))
    covered = np.zeros(meta[1], bool)
    for e, first, cnt, _ in chunks[:meta[0]]:
        assert 0 < cnt <= 128 and offs[e] <= first and first + cnt <= offs[e + 1]
        covered[first:first + cnt] = True
    assert covered.all() and meta[0] == np.ceil(counts / 128).sum()


def test_bounded_wait_runs_out_and_the_context_stays_usable():
    """A wait that nothing satisfies gives up after its limit, the host reads the code, and the next call is clean."""
    pkg = importlib.import_module("nano-vllm-moe_b200")
    Kn, L = kernels(), pkg._lib
    dev = torch.device("cuda", 0)
    assert Kn.read_status(dev) == 0
    ws = Kn.workspace(dev, L.WS_HEADER_BYTES)
    t0 = torch.cuda.Event(enable_timing=True); t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    L.raise_for(L.load().fp8lin_debug_wait_timeout(ws.data_ptr(), 3000, torch.cuda.current_stream().cuda_stream), "probe")
    t1.record()
    torch.cuda.synchronize()
    assert 0.5 < t0.elapsed_time(t1) < 500.0                 # about 3 ms of clock64 at the SM clock, not a second
    with pytest.raises(RuntimeError, match="bounded wait"):
        Kn.read_status(dev)
    assert Kn.read_status(dev) == 0                          # reading cleared it
    c = O.make_case(5, 130, 448, 576)
    from helpers import oracle_linear, run_linear, upload_case
    y = run_linear("fp8_w8a8_static", upload_case(c))
    assert_parity(y, oracle_linear("fp8_w8a8_static", c), "after a timed-out wait")
    assert Kn.read_status(dev) == 0
    assert L.load().fp8lin_debug_wait_timeout(ws.data_ptr(), 0, None) == L.ERR_ARG


def test_graph_captured_before_the_scratch_grows_still_replays_correctly():
    """A CUDA graph holds the address of the scratch it was captured with; a later, larger eager call on the same
    stream makes the scratch grow.  The old buffer is retired, not freed, so the replay still computes the same bits."""
    Kn = kernels()
    small = O.make_case(77, 256, 2048, 1024)        # quantised rows + cluster split-K live in scratch
    from helpers import oracle_linear, upload_case
    d = upload_case(small)
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        want = Kn.launch_w8a8_gemm(d["x"], d["w_nk"], d["input_scale"], d["w_scale"], d["bias"]).clone()
        torch.cuda.synchronize()
        out = torch.empty_like(want)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=side):
            Kn.launch_w8a8_gemm(d["x"], d["w_nk"], d["input_scale"], d["w_scale"], d["bias"], out=out)
        big = upload_case(O.make_case(78, 3000, 2048, 512))
        y_big = Kn.launch_w8a8_gemm(big["x"], big["w_nk"], big["input_scale"], big["w_scale"], big["bias"])   # grows the scratch
        filler = [torch.full((1 << 20,), 0x7F, dtype=torch.uint8, device="cuda") for _ in range(8)]       # would land in freed memory
        out.fill_(float("nan"))
        g.replay()
        torch.cuda.synchronize()
        assert torch.equal(out, want)
        del filler, y_big
        # growing inside a capture would record an allocation and a fill: refused with a clear message
        raised = []
        g2 = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g2, stream=side):
            out.add_(0)                                   # (keeps the captured graph non-empty)
            try:
                Kn.workspace(torch.device("cuda", 0), 1 << 30)
            except RuntimeError as exc:
                raised.append(str(exc))
        assert raised and "capture" in raised[0]
    assert_parity(from_bf16(want), oracle_linear("fp8_w8a8_static", small), "graph replay")


# (ranks, rows, K per rank, N): the last two are the 8-rank shards of the 7B down and o_proj layers at 16384 rows
BANDED = [(3, 1000, 256, 264), (8, 1000, 448, 576), (5, 4100, 1408, 520), (8, 16384, 2368, 3584), (8, 16384, 448, 3584)]


@pytest.mark.parametrize("tp,rows,k,n", BANDED)
def test_row_parallel_bands_of_many_ranks_emulated_on_one_gpu(tp, rows, k, n):
    """The reduce-scatter epilogue and the slot sum of RowParallelLinear at rank counts no box offered, with every
    rank's buffer in this GPU's memory and the ranks run one after the other: rank r's GEMM stores band d of its
    partial result into slot r of rank d's buffer, rank d adds its slots in order and stores the band to every
    rank's output.  Must equal, bit for bit, the plain GEMMs' bf16 partials added in rank order in fp32."""
    Kn = kernels()
    cases = [big_case(31 * r + tp + k, rows, k, n) for r in range(tp)]
    in_scale = cases[0]["input_scale"]
    band = -(-(-(-rows // tp)) // 32) * 32                    # rows per band as the layer rounds them
    slot = band * n
    bufs = [torch.full((tp * slot + rows * n,), float("nan"), dtype=torch.bfloat16, device="cuda") for _ in range(tp)]
    for r, d in enumerate(cases):
        dst = [bufs[o].data_ptr() + r * slot * 2 for o in range(tp)]
        Kn.launch_w8a8_reduce_scatter(d["x"], d["w_nk"], in_scale, d["w_scale"], d["bias"] if r == 0 else None, dst, n, band)
    ys = [b.data_ptr() + tp * slot * 2 for b in bufs]
    for r in range(tp):
        mine = max(0, min(band, rows - r * band))
        Kn.sum_slots_gather(bufs[r].data_ptr(), tp, slot, n, ys, n, r * band, mine, n, torch.device("cuda", 0))
    torch.cuda.synchronize()
    want = torch.zeros((rows, n), dtype=torch.float32, device="cuda")
    for r, d in enumerate(cases):
        want += Kn.launch_w8a8_gemm(d["x"], d["w_nk"], in_scale, d["w_scale"], d["bias"] if r == 0 else None).float()
    want = want.to(torch.bfloat16)
    for r in range(tp):
        got = bufs[r][tp * slot:].view(rows, n)
        assert torch.equal(got, want), f"rank {r}: {(got != want).sum().item()} elements differ"
    # and the sum against the oracle on sampled rows and columns
    rng = np.random.default_rng(rows + n)
    ri, ci = sample(rows, 24, rng), sample(n, 96, rng)
    ref = np.zeros((len(ri), len(ci)), dtype=np.float32)
    for r, d in enumerate(cases):
        x = from_bf16(d["x"][torch.from_numpy(ri).cuda()])
        ct = torch.from_numpy(ci).cuda()
        b = from_bf16(d["bias"][ct]) if r == 0 else None
        ref += O.linear_w8a8(x, d["q"][ct].cpu().numpy(), d["w_scale"][ct].cpu().numpy(), np.float32(in_scale.item()), b)
    got = from_bf16(bufs[0][tp * slot:].view(rows, n)[torch.from_numpy(ri).cuda()][:, torch.from_numpy(ci).cuda()])
    assert_parity(got, O.bf16_round(ref), f"{tp} ranks {rows}x{k}x{n}", ulps=float(tp))
