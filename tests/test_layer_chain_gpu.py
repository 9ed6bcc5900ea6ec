"""One decode token through a full-attention layer and its feed-forward block, issued as the reference
issues it (RunFullBlock and RunFfn, src/models/qwen3_5/trunk.cpp:268-470 of the reference: rmsnorm, the q+gate /
k / v projections, qgate_split, per-head rmsnorm, mrope, the cache append, attention, sigmoid_gate, the
output projection, add, rmsnorm, gate / up, silu_mul, down, add), launch by launch and through the deferred
queue (which folds the norms and adds into the projections and replays the sequence as a CUDA graph), with
fp32, fp16 and int8 caches.  Every step of the CPU oracle is bit-equal to the reference's *Ref function, so
the chain is the reference's host arithmetic for the layer; synthetic Q4_K weights stand in for a checkpoint."""
import numpy as np
import pytest

from tessera_b200 import synth
from tessera_b200.backend import KernelLaunch
from tessera_b200.project import Q4K, Projector

from conftest import rel_err

pytestmark = pytest.mark.gpu

EPS = 1e-6
HIDDEN, HEADS, KV_HEADS, HEAD_DIM, FFN = 1024, 8, 2, 128, 2048
Q_DIM, KV_DIM = HEADS * HEAD_DIM, KV_HEADS * HEAD_DIM
ROPE_DIM, SECTIONS, THETA = 64, (11, 11, 10), 1e7
PRIOR, CAPACITY = 70, 128   # keys already in the cache; the token sits at position PRIOR


def bits(x):
    return int(np.float32(x).view(np.uint32))


class Layer:
    """Weights, the cache's earlier rows and the oracle's result for the token."""

    def __init__(self, oracle, cache, seed):
        g = np.random.default_rng(seed)
        self.cache = cache
        self.x = g.standard_normal(HIDDEN).astype(np.float32)
        self.w = {name: synth.q4k_weights(n, k, seed=seed, index=i) for i, (name, n, k) in enumerate(
            [("q", 2 * Q_DIM, HIDDEN), ("k", KV_DIM, HIDDEN), ("v", KV_DIM, HIDDEN), ("o", HIDDEN, Q_DIM),
             ("gate", FFN, HIDDEN), ("up", FFN, HIDDEN), ("down", HIDDEN, FFN)])}
        self.norm = {name: (1.0 + 0.1 * g.standard_normal(n)).astype(np.float32)
                     for name, n in [("attn", HIDDEN), ("q", HEAD_DIM), ("k", HEAD_DIM), ("ffn", HIDDEN)]}
        self.pos = np.array([[PRIOR, PRIOR, PRIOR]], dtype=np.uint64)
        prior_k = g.standard_normal((PRIOR, KV_DIM)).astype(np.float32)
        prior_v = g.standard_normal((PRIOR, KV_DIM)).astype(np.float32)
        self.prior = self.encode(oracle, prior_k), self.encode(oracle, prior_v)
        self.want = self.reference(oracle)

    def encode(self, oracle, rows):
        """Rows of the cache in its format: (bytes per row, scales or None)."""
        if self.cache == "f32":
            return rows.copy(), None
        if self.cache == "f16":
            return rows.astype(np.float16), None
        codes, scale = oracle.quantize_rows(0, rows)
        return codes, scale

    def project(self, oracle, name, a):
        n, k = {"q": (2 * Q_DIM, HIDDEN), "k": (KV_DIM, HIDDEN), "v": (KV_DIM, HIDDEN), "o": (HIDDEN, Q_DIM),
                "gate": (FFN, HIDDEN), "up": (FFN, HIDDEN), "down": (HIDDEN, FFN)}[name]
        return oracle.gemm_q4k(a.reshape(1, k), self.w[name], 1, n, k).reshape(-1)

    def reference(self, oracle):
        o, st = oracle, {}
        xn = o.rmsnorm(self.x.reshape(1, -1), self.norm["attn"], EPS)
        q, gate = o.qgate_split(self.project(o, "q", xn), HEADS, HEAD_DIM, 1)
        kf, vf = self.project(o, "k", xn), self.project(o, "v", xn)
        q = o.rmsnorm(q.reshape(HEADS, HEAD_DIM), self.norm["q"], EPS).reshape(-1)
        kf = o.rmsnorm(kf.reshape(KV_HEADS, HEAD_DIM), self.norm["k"], EPS).reshape(-1)
        q = o.mrope(q, self.pos, 1, HEADS, HEAD_DIM, ROPE_DIM, *SECTIONS, float(np.float32(THETA)))
        kf = o.mrope(kf, self.pos, 1, KV_HEADS, HEAD_DIM, ROPE_DIM, *SECTIONS, float(np.float32(THETA)))
        (pk, pks), (pv, pvs) = self.prior
        (nk, nks), (nv, nvs) = self.encode(o, kf.reshape(1, -1)), self.encode(o, vf.reshape(1, -1))
        keys, values = np.concatenate([pk, nk]), np.concatenate([pv, nv])
        fmt = {"f32": 0, "f16": 1, "q8": 2}[self.cache]
        ks = None if pks is None else np.concatenate([pks, nks])
        vs = None if pvs is None else np.concatenate([pvs, nvs])
        kbytes = keys.view(np.uint8) if self.cache == "f16" else keys
        vbytes = values.view(np.uint8) if self.cache == "f16" else values
        attn = o.attention(fmt, q, kbytes, vbytes, 1, PRIOR + 1, HEADS, KV_HEADS, HEAD_DIM, PRIOR, 0, True, ks, vs).reshape(-1)
        attn = o.sigmoid_gate(attn, gate)
        x1 = o.add(self.x, self.project(o, "o", attn))
        xn2 = o.rmsnorm(x1.reshape(1, -1), self.norm["ffn"], EPS)
        act = o.silu_mul(self.project(o, "gate", xn2), self.project(o, "up", xn2))
        x2 = o.add(x1, self.project(o, "down", act))
        st.update(q=q, kf=kf, attn=attn, x1=x1, x2=x2)
        return st


class DeviceLayer:
    """The device buffers of the layer state (Qwen35State) and the reference's launch sequence."""

    def __init__(self, backend, layer):
        b, self.backend, self.layer = backend, backend, layer
        self.w = {k: b.upload(v) for k, v in layer.w.items()}
        self.norm = {k: b.upload(v) for k, v in layer.norm.items()}
        self.pos = b.upload(layer.pos)
        f = lambda n: b.AllocateBuffer(n * 4)
        self.x, self.xn, self.fused, self.q, self.gate = f(HIDDEN), f(HIDDEN), f(2 * Q_DIM), f(Q_DIM), f(Q_DIM)
        self.kf, self.vf, self.attn, self.proj = f(KV_DIM), f(KV_DIM), f(Q_DIM), f(HIDDEN)
        self.g, self.u, self.act = f(FFN), f(FFN), f(FFN)
        esz = {"f32": 4, "f16": 2, "q8": 1}[layer.cache]
        self.row_bytes = KV_DIM * esz
        self.k, self.v = b.AllocateBuffer(CAPACITY * self.row_bytes), b.AllocateBuffer(CAPACITY * self.row_bytes)
        self.ks, self.vs = f(CAPACITY), f(CAPACITY)
        self.kv_scratch, self.scale_scratch = b.AllocateBuffer(self.row_bytes), f(1)
        self.reset()

    def reset(self):
        b, (pk, pks), (pv, pvs) = self.backend, *self.layer.prior
        b.CopyH2D(self.x, self.layer.x)
        b.CopyH2D(self.k, pk.view(np.uint8).reshape(-1))
        b.CopyH2D(self.v, pv.view(np.uint8).reshape(-1))
        if pks is not None:
            b.CopyH2D(self.ks, pks)
            b.CopyH2D(self.vs, pvs)
        b.Synchronize()

    def launch(self, name, buffers, scalars):
        self.backend.LaunchKernel(self.backend.LoadKernel(name), KernelLaunch(buffers=buffers, scalars=scalars))

    def project(self, proj, name, a, out, n, k):
        proj.ProjectBatch(Q4K, a, self.w[name], out, 1, n, k)

    def append(self, src, cache, scales):
        """AppendKvRows (src/core/decode_internal.hpp:520-640): fp32 rows are copied, fp16 rows cast, int8 rows quantised."""
        b, c = self.backend, self.layer.cache
        if c == "f32":
            b.CopyD2D(src, 0, cache, PRIOR * self.row_bytes, self.row_bytes)
            return
        if c == "f16":
            self.launch("cast_f32_f16", [src, self.kv_scratch], [KV_DIM])
        else:
            self.launch("quantize_q8", [src, self.kv_scratch, self.scale_scratch], [1, KV_DIM])
            b.CopyD2D(self.scale_scratch, 0, scales, PRIOR * 4, 4)
        b.CopyD2D(self.kv_scratch, 0, cache, PRIOR * self.row_bytes, self.row_bytes)

    def issue(self, proj):
        L = self.launch
        L("rmsnorm", [self.x, self.norm["attn"], self.xn], [1, HIDDEN, bits(EPS)])
        self.project(proj, "q", self.xn, self.fused, 2 * Q_DIM, HIDDEN)
        L("qgate_split", [self.fused, self.q, self.gate], [HEADS, HEAD_DIM, 1])
        self.project(proj, "k", self.xn, self.kf, KV_DIM, HIDDEN)
        self.project(proj, "v", self.xn, self.vf, KV_DIM, HIDDEN)
        L("rmsnorm", [self.q, self.norm["q"], self.q], [HEADS, HEAD_DIM, bits(EPS)])
        L("rmsnorm", [self.kf, self.norm["k"], self.kf], [KV_HEADS, HEAD_DIM, bits(EPS)])
        L("mrope", [self.q, self.pos], [1, HEADS, HEAD_DIM, ROPE_DIM, bits(THETA), *SECTIONS])
        L("mrope", [self.kf, self.pos], [1, KV_HEADS, HEAD_DIM, ROPE_DIM, bits(THETA), *SECTIONS])
        self.append(self.kf, self.k, self.ks)
        self.append(self.vf, self.v, self.vs)
        rows = PRIOR + 1
        if self.layer.cache == "q8":
            L("attention_q8", [self.q, self.k, self.v, self.ks, self.vs, self.attn],
              [1, rows, HEADS, KV_HEADS, HEAD_DIM, PRIOR, 0, 0, 0])
        else:
            L("attention", [self.q, self.k, self.v, self.attn],
              [1, rows, HEADS, KV_HEADS, HEAD_DIM, PRIOR, 0, 0, int(self.layer.cache == "f16"), 1])
        L("sigmoid_gate", [self.attn, self.gate, self.attn], [Q_DIM])
        self.project(proj, "o", self.attn, self.proj, HIDDEN, Q_DIM)
        L("add", [self.x, self.proj, self.x], [HIDDEN])
        L("rmsnorm", [self.x, self.norm["ffn"], self.xn], [1, HIDDEN, bits(EPS)])
        self.project(proj, "gate", self.xn, self.g, FFN, HIDDEN)
        self.project(proj, "up", self.xn, self.u, FFN, HIDDEN)
        L("silu_mul", [self.g, self.u, self.act], [FFN])
        self.project(proj, "down", self.act, self.proj, HIDDEN, FFN)
        L("add", [self.x, self.proj, self.x], [HIDDEN])

    def check(self):
        b, want = self.backend, self.layer.want
        b.Synchronize()
        assert rel_err(b.download(self.q, np.float32, Q_DIM), want["q"]) < 1e-4
        assert rel_err(b.download(self.kf, np.float32, KV_DIM), want["kf"]) < 1e-4
        assert rel_err(b.download(self.attn, np.float32, Q_DIM), want["attn"]) < 2e-3
        assert rel_err(b.download(self.x, np.float32, HIDDEN), want["x2"]) < 2e-3


@pytest.mark.parametrize("cache", ["f32", "f16", "q8"])
def test_full_attention_layer_launch_by_launch(backend, oracle, cache):
    dev = DeviceLayer(backend, Layer(oracle, cache, seed=500))
    dev.issue(Projector(backend))
    dev.check()


@pytest.mark.parametrize("cache", ["f32", "q8"])
def test_full_attention_layer_through_the_deferred_queue(backend, oracle, cache):
    """The same sequence queued: the norms and adds fold into the projections, the cache copies sit between
    the launches, the whole token replays as a graph from its second appearance; the buffers must not change."""
    dev = DeviceLayer(backend, Layer(oracle, cache, seed=501))
    proj = Projector(backend)
    backend.Synchronize()
    backend.SetDeferred(1)
    try:
        for rep in range(3):   # the third pass replays what the second captured
            dev.reset()
            api0, dev0, graphs0 = backend.LaunchStats()
            dev.issue(proj)
            backend.Synchronize()
            api1, dev1, graphs1 = backend.LaunchStats()
            # the cache rows' copies wait in the queue with the launches, so the token is one queue:
            # fewer kernels than launches (norms and adds ride in the projections), one graph from its third run on
            assert dev1 - dev0 < api1 - api0
            if rep == 2:
                assert graphs1 - graphs0 == 1
            dev.check()
    finally:
        backend.SetDeferred(0)


# ---- a linear-attention (gated delta rule) layer, src/models/qwen3_5/trunk.cpp:715-785 of the reference
K_HEADS, V_HEADS, HEAD_K, HEAD_V, WIDTH = 4, 8, 128, 128, 4
KEY_DIM, VALUE_DIM = K_HEADS * HEAD_K, V_HEADS * HEAD_V
CONV_DIM, FACTOR = 2 * KEY_DIM + VALUE_DIM, V_HEADS // K_HEADS


class LinearLayer:
    def __init__(self, oracle, seed):
        g = np.random.default_rng(seed)
        self.x = g.standard_normal(HIDDEN).astype(np.float32)
        self.w = {name: synth.q4k_weights(n, k, seed=seed, index=i) for i, (name, n, k) in enumerate(
            [("qkv", CONV_DIM, HIDDEN), ("z", VALUE_DIM, HIDDEN), ("out", HIDDEN, VALUE_DIM)])}
        # the per-head gate projections are fp32 tensors (gemm_f32)
        self.w_alpha = (g.standard_normal((V_HEADS, HIDDEN)) * 0.05).astype(np.float32)
        self.w_beta = (g.standard_normal((V_HEADS, HIDDEN)) * 0.05).astype(np.float32)
        self.norm = (1.0 + 0.1 * g.standard_normal(HIDDEN)).astype(np.float32)
        self.ssm_norm = (1.0 + 0.1 * g.standard_normal(HEAD_V)).astype(np.float32)
        self.conv_w = (g.standard_normal((CONV_DIM, WIDTH)) * 0.02).astype(np.float32)
        self.a_log = (-np.exp(g.standard_normal(V_HEADS))).astype(np.float32)
        self.dt = g.standard_normal(V_HEADS).astype(np.float32)
        self.hist = g.standard_normal(CONV_DIM * (WIDTH - 1)).astype(np.float32)
        self.state = (g.standard_normal(V_HEADS * HEAD_K * HEAD_V) * 0.1).astype(np.float32)
        self.want = self.reference(oracle)

    def reference(self, o):
        xn = o.rmsnorm(self.x.reshape(1, -1), self.norm, EPS)
        qkv = o.gemm_q4k(xn, self.w["qkv"], 1, CONV_DIM, HIDDEN).reshape(-1)
        z = o.gemm_q4k(xn, self.w["z"], 1, VALUE_DIM, HIDDEN).reshape(-1)
        beta_raw = o.gemm_dense(False, xn, self.w_beta, 1, V_HEADS, HIDDEN)
        alpha_raw = o.gemm_dense(False, xn, self.w_alpha, 1, V_HEADS, HIDDEN)
        alpha, beta = o.ssm_gate(self.a_log, self.dt, alpha_raw, beta_raw)
        q, k, v, hist, _ = o.conv1d_state(qkv, self.conv_w, self.hist, CONV_DIM, WIDTH, KEY_DIM, 0, 1)
        q = o.l2norm(q.reshape(K_HEADS, HEAD_K), 1e-6, np.float32(1.0 / np.sqrt(float(HEAD_K)))).reshape(-1)
        k = o.l2norm(k.reshape(K_HEADS, HEAD_K), 1e-6, np.float32(1.0)).reshape(-1)
        q_exp, k_exp = o.repeat_heads(q, V_HEADS, HEAD_K, FACTOR), o.repeat_heads(k, V_HEADS, HEAD_K, FACTOR)
        state, core = o.delta_step_heads(self.state, k_exp, v, q_exp, alpha.reshape(-1), beta.reshape(-1), V_HEADS, HEAD_K, HEAD_V)
        out = o.rmsnorm_gated(core.reshape(V_HEADS, HEAD_V), self.ssm_norm, z.reshape(V_HEADS, HEAD_V), EPS).reshape(-1)
        x1 = o.add(self.x, o.gemm_q4k(out.reshape(1, -1), self.w["out"], 1, HIDDEN, VALUE_DIM).reshape(-1))
        return dict(hist=hist, state=state, core=core, x1=x1)


def issue_linear(backend, proj, layer, d):
    def L(name, buffers, scalars):
        backend.LaunchKernel(backend.LoadKernel(name), KernelLaunch(buffers=buffers, scalars=scalars))
    L("rmsnorm", [d["x"], d["norm"], d["xn"]], [1, HIDDEN, bits(EPS)])
    proj.ProjectBatch(Q4K, d["xn"], d["w_qkv"], d["qkv"], 1, CONV_DIM, HIDDEN)
    proj.ProjectBatch(Q4K, d["xn"], d["w_z"], d["z"], 1, VALUE_DIM, HIDDEN)
    L("gemm_f32", [d["xn"], d["w_beta"], d["beta_raw"]], [1, V_HEADS, HIDDEN])
    L("gemm_f32", [d["xn"], d["w_alpha"], d["alpha_raw"]], [1, V_HEADS, HIDDEN])
    L("ssm_gate", [d["a_log"], d["dt"], d["alpha_raw"], d["beta_raw"], d["alpha"], d["beta"]], [V_HEADS, 1])
    L("conv1d_state", [d["qkv"], d["conv_w"], d["hist"], d["q"], d["k"], d["v"], d["hist"]], [CONV_DIM, WIDTH, KEY_DIM, 0, 1, 0])
    L("l2norm", [d["q"], d["q"]], [K_HEADS, HEAD_K, bits(1e-6), bits(1.0 / np.sqrt(float(HEAD_K)))])
    L("l2norm", [d["k"], d["k"]], [K_HEADS, HEAD_K, bits(1e-6), bits(1.0)])
    L("repeat_heads", [d["q"], d["q_exp"]], [V_HEADS, HEAD_K, FACTOR, 1])
    L("repeat_heads", [d["k"], d["k_exp"]], [V_HEADS, HEAD_K, FACTOR, 1])
    L("delta_step_heads", [d["state"], d["k_exp"], d["v"], d["q_exp"], d["core"], d["alpha"], d["beta"]],
      [V_HEADS, HEAD_K, HEAD_V, 1, 0, 0, 0])
    L("rmsnorm_gated", [d["core"], d["ssm_norm"], d["z"], d["out"]], [V_HEADS, HEAD_V, bits(EPS), 0, 0])
    proj.ProjectBatch(Q4K, d["out"], d["w_out"], d["proj"], 1, HIDDEN, VALUE_DIM)
    L("add", [d["x"], d["proj"], d["x"]], [HIDDEN])


@pytest.mark.parametrize("deferred", [0, 1])
def test_linear_attention_layer(backend, oracle, deferred):
    layer = LinearLayer(oracle, seed=600)
    up, f = backend.upload, lambda n: backend.AllocateBuffer(n * 4)
    d = dict(x=up(layer.x), norm=up(layer.norm), ssm_norm=up(layer.ssm_norm), conv_w=up(layer.conv_w), a_log=up(layer.a_log),
             dt=up(layer.dt), hist=up(layer.hist), state=up(layer.state), w_alpha=up(layer.w_alpha), w_beta=up(layer.w_beta),
             w_qkv=up(layer.w["qkv"]), w_z=up(layer.w["z"]), w_out=up(layer.w["out"]),
             xn=f(HIDDEN), qkv=f(CONV_DIM), z=f(VALUE_DIM), beta_raw=f(V_HEADS), alpha_raw=f(V_HEADS), alpha=f(V_HEADS),
             beta=f(V_HEADS), q=f(KEY_DIM), k=f(KEY_DIM), v=f(VALUE_DIM), q_exp=f(V_HEADS * HEAD_K), k_exp=f(V_HEADS * HEAD_K),
             core=f(VALUE_DIM), out=f(VALUE_DIM), proj=f(HIDDEN))
    backend.Synchronize()
    backend.SetDeferred(deferred)
    try:
        issue_linear(backend, Projector(backend), layer, d)
        backend.Synchronize()
    finally:
        backend.SetDeferred(0)
    want = layer.want
    assert rel_err(backend.download(d["hist"], np.float32, layer.hist.size), want["hist"]) < 1e-6
    assert rel_err(backend.download(d["state"], np.float32, layer.state.size), want["state"]) < 1e-4
    assert rel_err(backend.download(d["core"], np.float32, VALUE_DIM), want["core"]) < 1e-4
    assert rel_err(backend.download(d["x"], np.float32, HIDDEN), want["x1"]) < 2e-3
