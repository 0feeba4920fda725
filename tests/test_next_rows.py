"""The rows either side of the hot path: the prefill chunk policy, the on-disk NVFP4 triple, and
silu_mul between gate/up and down (CPU parts here; the GPU parts are marked gpu)."""
import numpy as np
import pytest

import lex_gpu_b200 as L
from lex_gpu_b200 import checkpoint, inputs
from oracle import oracle as O


def _chunks_restated(tokens, limit=0, gemm_ok=True):
    """Runner::chunk + prefill_limit (crates/lex-rt/src/qwen_run.rs:2478-2501), restated."""
    sizes, max_batch = [512, 256, 128, 64, 32, 16], 8
    lim = next((g for g in sizes if g <= (limit or 512)), max_batch) if gemm_ok else max_batch
    out, left = [], tokens
    while left:
        take = next((g for g in sizes if gemm_ok and g <= lim and g <= left), min(left, max_batch))
        out.append(take)
        left -= take
    return out


def test_prefill_chunk_policy_matches_the_runner():
    for tokens in list(range(0, 70)) + [127, 128, 129, 511, 512, 513, 1000, 2048, 4095, 8191]:
        for limit in (0, 512, 300, 128, 16, 9):
            assert L.prefill_chunks(tokens, limit) == _chunks_restated(tokens, limit), (tokens, limit)
        assert L.prefill_chunks(tokens, gemm_ok=False) == _chunks_restated(tokens, gemm_ok=False)
    assert L.prefill_chunks(1000) == [512, 256, 128, 64, 32, 8]
    assert sum(L.prefill_chunks(8191)) == 8191


def test_nvfp4_blob_round_trip_and_nibble_order(tmp_path):
    wq, ws, wg = inputs.make_weights(48, 256, seed_base=4)
    path = tmp_path / "blob.safetensors"
    checkpoint.write_nvfp4(path, {"blk.0.ffn_gate.weight": (wq, ws, 0.75), "blk.0.ffn_up.weight": (wq[::-1].copy(), ws, 1.5)})
    assert set(checkpoint.tensor_names(path)) >= {"blk.0.ffn_gate.weight", "blk.0.ffn_gate.weight.scale"}
    q2, s2, g2 = checkpoint.read_nvfp4(path, "blk.0.ffn_gate.weight")
    assert np.array_equal(q2, wq) and np.array_equal(s2, ws) and np.array_equal(g2, np.full(48, 0.75, np.float32))
    # the file's own statement of the order: value k of a little-endian u32 word is bits 4k..4k+3
    # (scripts/qwen_nvfp4.py:75-82) - the same codes the operator's nibble rule gives (interp.rs:650)
    words = q2.view("<u4")
    nib = np.empty((48, 256), dtype=np.uint8)
    for kk in range(8):
        nib[:, kk::8] = (words >> (4 * kk)) & 0xF
    assert np.array_equal(nib, O.np_codes(q2))
    with pytest.raises(KeyError):
        checkpoint.read_nvfp4(path, "blk.0.ffn_down.weight")


def test_silu_mul_oracle_matches_the_formula():
    """lex_front::llama tests::silu_mul_matches_the_formula (crates/lex-front/src/llama.rs:1412-1429)."""
    rng = np.random.Generator(np.random.PCG64(1))
    g, u = rng.standard_normal(4096).astype(np.float32) * 4, rng.standard_normal(4096).astype(np.float32)
    want = (g.astype(np.float64) / (1.0 + np.exp(-g.astype(np.float64))) * u).astype(np.float32)
    assert O.max_rel_err(O.np_silu_mul(g, u), want) < 1e-6


@pytest.fixture(scope="module")
def gpu():
    from lex_gpu_b200 import build
    build.build()
    g = L.Gpu(0)
    yield g
    g.close()


@pytest.mark.gpu
def test_silu_mul_on_device(gpu):
    rng = np.random.Generator(np.random.PCG64(2))
    rows, cols = 37, 1024
    g = (rng.standard_normal((rows, cols)) * 6).astype(np.float32)
    u = rng.standard_normal((rows, cols)).astype(np.float32) * 3
    g[0, :4] = [0.0, -0.0, 88.0, -104.0]
    gb, ub = gpu.upload(g), gpu.upload(u)
    o32, o16 = gpu.alloc(rows * cols * 4), gpu.alloc(rows * cols * 2)
    gpu.silu_mul(rows, cols, gb, ub, o32, out_f16=False)
    gpu.silu_mul(rows, cols, gb, ub, o16, out_f16=True)
    got32 = gpu.download(o32, np.float32, (rows, cols))
    got16 = gpu.download(o16, np.float16, (rows, cols))
    want = O.np_silu_mul(g, u)
    assert O.max_rel_err(got32, want) < 1e-6                       # the reference's own tolerance
    # f16 output: the same value rounded once; at most one f16 step where the f32 values differ by an ulp
    d = np.abs(got16.astype(np.float32) - want.astype(np.float16).astype(np.float32))
    assert np.all(d <= np.abs(want) * 2.0 ** -10 + 1e-7)
    with pytest.raises(L.LexbError):
        gpu.silu_mul(rows, 1022, gb, ub, o32, out_f16=False)


@pytest.mark.gpu
def test_mlp_block_gate_up_fused_silu_down(gpu, tmp_path):
    """One MLP block as lex-rt runs it (crates/lex-rt/src/qwen_run.rs:3165-3189), from a synthetic blob:
    gate and up in ONE gemm_fp4 launch over their rows concatenated, silu_mul to f16, down with the
    residual - every stage against the oracle."""
    m, hidden, ffn = 96, 512, 1024
    rng = np.random.Generator(np.random.PCG64(3))
    mats = {}
    for i, (name, n, k) in enumerate([("gate", ffn, hidden), ("up", ffn, hidden), ("down", hidden, ffn)]):
        wq, ws, _ = inputs.make_weights(n, k, seed_base=30 + i)
        mats[name] = (wq, ws, [0.02, 0.03, 0.01][i])
    path = tmp_path / "mlp.safetensors"
    checkpoint.write_nvfp4(path, {f"blk.0.ffn_{k}.weight": v for k, v in mats.items()})
    W = {k: checkpoint.read_nvfp4(path, f"blk.0.ffn_{k}.weight") for k in mats}
    x = inputs.make_x(m, hidden, seed_base=3)
    resid = rng.standard_normal((m, hidden)).astype(np.float32)

    # oracle
    yg = O.gemm_fp4(x, *W["gate"])
    yu = O.gemm_fp4(x, *W["up"])
    a16 = O.np_silu_mul(yg, yu, out_f16=True)
    want = O.gemm_fp4(a16, *W["down"], r=resid)

    # device: concatenated gate|up weights, one launch; silu_mul reads the two halves of its output
    cat = [np.concatenate([W["gate"][i], W["up"][i]], axis=0) for i in range(3)]
    qgu, qd = L.QBuf(gpu, *cat), L.QBuf(gpu, *W["down"])
    xb, rb = gpu.upload(x), gpu.upload(resid)
    ygu, act, yout = gpu.alloc(m * 2 * ffn * 4), gpu.alloc(m * ffn * 2), gpu.alloc(m * hidden * 4)
    p1, p2 = gpu.plan_gemm_fp4(m, 2 * ffn, hidden), gpu.plan_gemm_fp4(m, hidden, ffn, residual=True)
    gpu.run(p1, qgu.bind(xb, None, ygu))
    gpu.silu_mul(m, ffn, ygu, ygu, act, out_f16=True, gate_pitch=2 * ffn, up_offset=ffn, up_pitch=2 * ffn)
    gpu.run(p2, qd.bind(act, rb, yout))
    got_gu = gpu.download(ygu, np.float32, (m, 2 * ffn))
    got_act = gpu.download(act, np.float16, (m, ffn))
    got = gpu.download(yout, np.float32, (m, hidden))
    assert gpu.status_word() == 0
    e1, s1, r1 = O.err_of_scale(got_gu, np.concatenate([yg, yu], axis=1))
    assert s1 > 1e-3 and e1 <= 2e-3 and r1 <= 2e-3
    # silu_mul on the device's own gate/up: equal to the oracle's evaluation of the same inputs up to one f16 step
    a_dev_in = O.np_silu_mul(got_gu[:, :ffn], got_gu[:, ffn:], out_f16=True).astype(np.float32)
    assert np.all(np.abs(got_act.astype(np.float32) - a_dev_in) <= np.abs(a_dev_in) * 2.0 ** -10 + 1e-7)
    # down on the device's own activation, against the oracle on that same activation
    e2, s2, r2 = O.err_of_scale(got, O.gemm_fp4(got_act, *W["down"], r=resid))
    assert s2 > 1e-3 and e2 <= 2e-3 and r2 <= 2e-3
    # and the whole block against the oracle's chain, of scale (inputs of the last stage differ by f16 steps)
    e3, s3, _ = O.err_of_scale(got, want)
    assert s3 > 1e-3 and e3 <= 2e-3


@pytest.mark.gpu
@pytest.mark.parametrize("m,ffn,hidden,splits", [(96, 1024, 512, 0), (512, 768, 1024, 0), (700, 512, 2048, 2), (300, 640, 1280, 5)])
def test_gate_up_in_one_launch_with_silu_mul_in_the_epilogue(gpu, m, ffn, hidden, splits):
    """The three dispatches of crates/lex-rt/src/qwen_run.rs:3165-3183 (gate, up, silu_mul) as one launch: rows of
    gate and up interleaved at load, silu(gate) * up formed in the GEMM's epilogue (in the reduction launch when K
    is split) and written as the f16 activation.  Against (1) the same launch's f32 gate/up run through the
    interpreter's formula: equal up to one f16 step; (2) the oracle's whole chain, of scale."""
    x = inputs.make_x(m, hidden, seed_base=40)
    wg_, wu_ = inputs.make_weights(ffn, hidden, seed_base=41), inputs.make_weights(ffn, hidden, seed_base=42)
    # row scales that keep gate near the knee of the sigmoid
    wg_ = (wg_[0], wg_[1], (wg_[2] * np.float32(0.02)).astype(np.float32))
    wu_ = (wu_[0], wu_[1], (wu_[2] * np.float32(0.03)).astype(np.float32))
    qg, qu = L.QBuf(gpu, *wg_), L.QBuf(gpu, *wu_)
    qgu = L.QBuf.gate_up(gpu, qg, qu)
    # the interleave itself: row 2j = gate j, 2j + 1 = up j, for all three arrays
    for dev, a, b, dt in ((qgu.wq, wg_[0], wu_[0], np.uint8), (qgu.ws, wg_[1], wu_[1], np.uint8), (qgu.wg, wg_[2], wu_[2], np.float32)):
        got = gpu.download(dev, dt, (2 * ffn,) + a.shape[1:])
        assert np.array_equal(got[0::2], a) and np.array_equal(got[1::2], b)
    xb = gpu.upload(x)
    pipe = gpu.plan_gemm_fp4(m, 2 * ffn, hidden, kernel=3, k_splits=splits)
    act, ygu = gpu.alloc(m * ffn * 2), gpu.alloc(m * 2 * ffn * 4)
    gpu.memset(act, 0xFF)
    gpu.run_silu(pipe, xb, qgu.wq, qgu.ws, qgu.wg, act)
    gpu.run(pipe, qgu.bind(xb, None, ygu))
    got_act = gpu.download(act, np.float16, (m, ffn))
    got_gu = gpu.download(ygu, np.float32, (m, 2 * ffn))
    assert gpu.status_word() == 0
    assert np.isfinite(got_act.astype(np.float32)).all()
    same_inputs = O.np_silu_mul(got_gu[:, 0::2], got_gu[:, 1::2], out_f16=True).astype(np.float32)
    assert np.all(np.abs(got_act.astype(np.float32) - same_inputs) <= np.abs(same_inputs) * 2.0 ** -10 + 1e-7)
    want = O.np_silu_mul(O.gemm_fp4(x, *wg_), O.gemm_fp4(x, *wu_), out_f16=True).astype(np.float32)
    err, scale, rel = O.err_of_scale(got_act.astype(np.float32), want)
    print(f"  fused activation vs the oracle's chain: {err:.2e} of scale, {rel:.2e} per element")
    assert scale > 1e-3 and err <= 2e-3 and rel <= 2e-3
    with pytest.raises(L.LexbError):                      # a residual pipeline has no fused form
        gpu.run_silu(gpu.plan_gemm_fp4(m, 2 * ffn, hidden, residual=True, kernel=3), xb, qgu.wq, qgu.ws, qgu.wg, act)
    with pytest.raises(L.LexbError):                      # nor has the one-CTA kernel
        gpu.run_silu(gpu.plan_gemm_fp4(m, 2 * ffn, hidden, kernel=2), xb, qgu.wq, qgu.ws, qgu.wg, act)


@pytest.mark.gpu
@pytest.mark.parametrize("splits", [1, 3])
def test_fused_activation_gathered_into_every_ranks_buffer(gpu, splits):
    """The n-sharded form: this 'rank' owns interleaved rows [n0, n0 + n) and stores its columns of the f16
    activation into every rank's buffer (three buffers on one GPU stand for the ranks)."""
    m, ffn_local, hidden, ffn_total, col0 = 300, 256, 1536, 1024, 384
    x = inputs.make_x(m, hidden, seed_base=50)
    wg_, wu_ = inputs.make_weights(ffn_local, hidden, seed_base=51), inputs.make_weights(ffn_local, hidden, seed_base=52)
    wg_ = (wg_[0], wg_[1], (wg_[2] * np.float32(0.02)).astype(np.float32))
    wu_ = (wu_[0], wu_[1], (wu_[2] * np.float32(0.03)).astype(np.float32))
    qgu = L.QBuf.gate_up(gpu, L.QBuf(gpu, *wg_), L.QBuf(gpu, *wu_))
    xb = gpu.upload(x)
    pipe = gpu.plan_gemm_fp4(m, 2 * ffn_local, hidden, kernel=3, k_splits=splits)
    local = gpu.alloc(m * ffn_local * 2)
    gpu.run_silu(pipe, xb, qgu.wq, qgu.ws, qgu.wg, local)
    want = gpu.download(local, np.float16, (m, ffn_local))
    bufs = [gpu.alloc(m * ffn_total * 2) for _ in range(3)]
    for b in bufs:
        gpu.memset(b, 0xFF)
    gpu.run_silu_gather(pipe, xb, qgu.wq, qgu.ws, qgu.wg, [b.ptr for b in bufs], 2 * ffn_total, 2 * col0)
    assert gpu.status_word() == 0
    for b in bufs:
        full = gpu.download(b, np.uint16, (m, ffn_total))
        assert np.array_equal(full[:, col0:col0 + ffn_local], want.view(np.uint16))
        assert (full[:, :col0] == 0xFFFF).all() and (full[:, col0 + ffn_local:] == 0xFFFF).all()
    ref = O.np_silu_mul(O.gemm_fp4(x, *wg_), O.gemm_fp4(x, *wu_), out_f16=True).astype(np.float32)
    err, scale, rel = O.err_of_scale(want.astype(np.float32), ref)
    assert scale > 1e-3 and err <= 2e-3 and rel <= 2e-3


def test_ollama_store_manifest_and_sharded_reads(tmp_path, monkeypatch):
    """The store around the blobs (crates/lex-rt/src/qwen.rs:86-145): a manifest maps tensor names to blob files;
    a rank of an n-sharded run reads its own 128-row tiles only, and the slabs of all ranks tile the matrix."""
    mats = {}
    for i, (name, n, k) in enumerate([("blk.0.ffn_gate.weight", 1152, 256), ("blk.0.ffn_up.weight", 1152, 256), ("blk.0.ffn_down.weight", 256, 1152)]):
        wq, ws, _ = inputs.make_weights(n, k, seed_base=70 + i)
        mats[name] = (wq, ws, [0.02, 0.03, 0.5][i])
    checkpoint.write_store(tmp_path, "synthetic:27b", mats)
    st = checkpoint.Store.open("synthetic:27b", root=tmp_path)
    assert st.names() == sorted(mats) and st.has("blk.0.ffn_up.weight") and not st.has("nope")
    monkeypatch.setenv("OLLAMA_MODELS", str(tmp_path))             # the default root comes from the environment
    assert checkpoint.Store.open("synthetic:27b").names() == st.names()
    for name, (wq, ws, gs) in mats.items():
        full = st.nvfp4(name)
        assert np.array_equal(full[0], wq) and np.array_equal(full[1], ws) and np.all(full[2] == np.float32(gs))
    # 1152 rows = 9 tiles over 4 ranks: 3, 2, 2, 2 tiles; the spans are lexb_shard_rows' own
    name = "blk.0.ffn_gate.weight"
    spans = []
    for rank in range(4):
        wq, ws, wg, n0, n1 = st.nvfp4_shard(name, 4, rank)
        assert (n0, n1) == L.shard_rows(1152, 4, rank) == checkpoint.shard_span(1152, 4, rank)
        assert np.array_equal(wq, mats[name][0][n0:n1]) and np.array_equal(ws, mats[name][1][n0:n1]) and wg.shape == (n1 - n0,)
        spans.append((n0, n1))
    assert spans[0][0] == 0 and spans[-1][1] == 1152 and all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
    # gate and up of a rank, interleaved for the fused launch
    cols = []
    for rank in range(2):
        wq, ws, wg, j0, j1 = st.gate_up_shard("blk.0.ffn_gate.weight", "blk.0.ffn_up.weight", 2, rank)
        g, u = mats["blk.0.ffn_gate.weight"], mats["blk.0.ffn_up.weight"]
        assert np.array_equal(wq[0::2], g[0][j0:j1]) and np.array_equal(wq[1::2], u[0][j0:j1])
        assert np.array_equal(ws[0::2], g[1][j0:j1]) and np.array_equal(ws[1::2], u[1][j0:j1])
        assert np.all(wg[0::2] == np.float32(g[2])) and np.all(wg[1::2] == np.float32(u[2])) and (2 * (j1 - j0)) % 128 == 0
        cols.append((j0, j1))
    assert cols[0][0] == 0 and cols[0][1] == cols[1][0] and cols[1][1] == 1152
    # errors: a model that is not there, a manifest without named layers, rows outside the matrix
    with pytest.raises(FileNotFoundError):
        checkpoint.Store.open("missing", root=tmp_path)
    mdir = tmp_path / "manifests" / "registry.ollama.ai" / "library" / "empty"
    mdir.mkdir(parents=True)
    (mdir / "latest").write_text('{"layers": [{"digest": "sha256:1"}]}')
    with pytest.raises(ValueError):
        checkpoint.Store.open("empty", root=tmp_path)
    with pytest.raises(ValueError):
        st.nvfp4(name, (1024, 2048))
    with pytest.raises(KeyError):
        st.nvfp4("blk.9.missing")
