"""The package's own PrivateUse1 backend (torch device "applegpu") over DEVICE-memory buffers.

Follows the reference's acceptance tests for its C++ backend, python/tests/test_cpp_backend.py: allocation and
copies (:15-60), element-wise ops / mm / addmm (:63-140), nn.Linear and the MLP (:143-215), embedding, layer_norm,
gelu, softmax and views (:218-371), the GELU written out in Python (:373-393), and HuggingFace GPT-2 greedy
generation equal to the CPU's with and without a KV cache (:396-480) -- there on the released checkpoint, here on a
seeded random initialisation of the same architecture (no network). Unlike tests/test_gpu_privateuse1_shim.py,
which runs the reference's shim in the managed-memory mode its host memcpy needs, nothing here sets
APPLEGPU_HOST_VISIBLE: every pointer is device memory and every byte moves through the ABI's copy calls.
Each case is a child process: PrivateUse1 can be named once per process.
"""
import os
import subprocess
import sys
import textwrap

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

_PRELUDE = """
    import torch
    import torch.nn.functional as F
    from applegpu_runtime_b200 import torch_device, _lib
    torch_device.load()
    lib = _lib.load()
    dev = "applegpu"
    def close(a, b, tol=1e-5):
        a = a.cpu().double(); b = b.cpu().double()
        assert a.shape == b.shape, (a.shape, b.shape)
        return float((a - b).abs().max() / b.abs().max().clamp_min(1e-30)) <= tol
"""


def _source(*pieces):
    return "".join(textwrap.dedent(p) for p in (_PRELUDE,) + pieces)


def _run(*pieces, timeout=900):
    env = {k: v for k, v in os.environ.items() if k != "APPLEGPU_HOST_VISIBLE"}
    env["PYTHONPATH"] = ROOT + os.pathsep + env.get("PYTHONPATH", "")
    r = subprocess.run([sys.executable, "-c", _source(*pieces)], env=env, cwd=ROOT, capture_output=True, text=True, timeout=timeout)
    assert r.returncode == 0, r.stdout[-3000:] + "\n" + r.stderr[-6000:]
    return r.stdout


def test_extension_loads_and_fails_loudly_without_a_device():
    """CPU: the extension loads against the installed torch (every symbol resolves) and registers the device; with no
    GPU the first allocation raises instead of falling back to anything."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("covers the no-GPU error path")
    out = _run("""
        try:
            torch.empty(2, 3, device=dev)
        except RuntimeError as e:
            assert "applegpu" in str(e), e
            print("raised")
    """)
    assert out.strip() == "raised"


@pytest.mark.gpu
def test_copies_fills_and_views_on_device_memory():
    out = _run("""
        torch.manual_seed(0)
        assert lib.applegpu_host_visible() == 0
        t = torch.empty(3, 4, device=dev)
        assert t.device.type == "applegpu" and t.shape == (3, 4) and t.dtype == torch.float32
        for dt in (torch.float32, torch.float16, torch.bfloat16, torch.int32, torch.int64, torch.uint8, torch.bool):
            src = (torch.randn(5, 7) * 10).to(dt)
            assert torch.equal(src.to(dev).cpu(), src), dt
        src = torch.randn(6, 9)
        g = torch.empty(6, 9, device=dev); g.copy_(src)
        assert torch.equal(g.cpu(), src)
        # strided views share the storage; copies out of and into them run as strided copy kernels
        assert torch.equal(g.t().cpu(), src.t()) and torch.equal(g[1:4, 2:7].cpu(), src[1:4, 2:7])
        assert torch.equal(g.t().contiguous().cpu(), src.t().contiguous())
        assert torch.equal(g.view(3, 18).cpu(), src.view(3, 18)) and torch.equal(g.reshape(-1)[5:20].cpu(), src.reshape(-1)[5:20])
        h = torch.zeros(6, 9, device=dev)
        h[:, 3:5] = g[:, 0:2]
        ref = torch.zeros(6, 9); ref[:, 3:5] = src[:, 0:2]
        assert torch.equal(h.cpu(), ref)
        h.t()[2:4].copy_(torch.ones(2, 6))                      # host -> strided device view
        ref.t()[2:4].copy_(torch.ones(2, 6))
        assert torch.equal(h.cpu(), ref)
        # converting copies: device -> device cast kernel, host <-> device through the host's converter
        assert torch.equal(g.to(torch.float16).cpu(), src.to(torch.float16))
        assert torch.equal(g.to(torch.bfloat16).cpu(), src.to(torch.bfloat16))
        d16 = torch.empty(6, 9, device=dev, dtype=torch.float16); d16.copy_(src)
        assert torch.equal(d16.cpu(), src.half())
        out32 = torch.empty(6, 9); out32.copy_(d16)
        assert torch.equal(out32, src.half().float())
        # fills
        assert torch.equal(torch.zeros(4, 5, device=dev).cpu(), torch.zeros(4, 5))
        assert torch.equal(torch.ones(4, 5, device=dev, dtype=torch.int64).cpu(), torch.ones(4, 5, dtype=torch.int64))
        assert torch.equal(torch.full((3, 3), 2.5, device=dev, dtype=torch.bfloat16).cpu(), torch.full((3, 3), 2.5, dtype=torch.bfloat16))
        f = torch.randn(4, 6).to(dev); f[:, 1::2].fill_(7.0)
        assert bool((f.cpu()[:, 1::2] == 7.0).all()) and bool((f.cpu()[:, 0::2] != 7.0).all())
        f.zero_(); assert float(f.cpu().abs().sum()) == 0.0
        # scalars and resize_
        assert torch.tensor(3.25, device=dev).item() == 3.25 and torch.arange(10, device=dev)[7].item() == 7
        r = torch.arange(6, device=dev, dtype=torch.float32); r.resize_(3, 4)
        assert torch.equal(r.cpu().reshape(-1)[:6], torch.arange(6, dtype=torch.float32))
        e = torch.empty(0, 4, device=dev); assert e.cpu().shape == (0, 4)
        # clone / detach / storage sharing
        c = g.clone(); c.add_(1.0)
        assert torch.equal(g.cpu(), src) and close(c, src + 1.0)
        assert g.detach().data_ptr() == g.data_ptr() and g[2:].data_ptr() == g.data_ptr() + 2 * 9 * 4
        torch.applegpu.synchronize()
        print("ok", lib.applegpu_launch_count())
    """)
    assert out.strip().startswith("ok") and int(out.split()[1]) > 10


@pytest.mark.gpu
def test_aten_ops_route_to_the_device_kernels():
    out = _run("""
        import math
        torch.manual_seed(0)
        n0 = lib.applegpu_launch_count()
        a, b = torch.randn(33, 65), torch.randn(33, 65)
        ga, gb = a.to(dev), b.to(dev)
        assert close(ga + gb, a + b) and close(ga * gb, a * b) and close(ga - gb, a - b) and close(ga / gb, a / b)
        assert close(ga + gb[0], a + b[0]) and close(ga * gb[:, :1], a * b[:, :1])            # broadcasts
        assert close(ga * 2.5, a * 2.5) and close(ga / 4, a / 4) and close(1.0 + ga, 1.0 + a) and close(ga - 3, a - 3) and close(2.0 - ga, 2.0 - a)
        assert close(torch.add(ga, gb, alpha=0.5), torch.add(a, b, alpha=0.5))
        assert close(torch.relu(ga), torch.relu(a)) and close(-ga, -a) and close(torch.tanh(ga), torch.tanh(a), 1e-5) and close(ga.abs().sqrt(), a.abs().sqrt())
        assert close(torch.sigmoid(ga), torch.sigmoid(a)) and close(torch.exp(ga), torch.exp(a)) and close(ga ** 3, a ** 3) and close(torch.pow(ga, 2.0), a ** 2)
        assert close(F.gelu(ga), F.gelu(a), 1e-5) and close(F.gelu(ga, approximate="tanh"), F.gelu(a, approximate="tanh"), 1e-5)
        # the tanh form written out in Python (what HuggingFace's NewGELUActivation runs)
        new_gelu = lambda x: 0.5 * x * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (x + 0.044715 * torch.pow(x, 3.0))))
        assert close(new_gelu(ga), new_gelu(a), 1e-5)
        # matmul family
        m1, m2, bias = torch.randn(40, 24), torch.randn(24, 56), torch.randn(56)
        assert close(torch.mm(m1.to(dev), m2.to(dev)), m1 @ m2)
        w = torch.randn(56, 24)
        assert close(torch.addmm(bias.to(dev), m1.to(dev), w.to(dev).t()), torch.addmm(bias, m1, w.t()))
        assert close(torch.addmm(torch.randn(40, 56).to(dev) * 0 + 1.0, m1.to(dev), m2.to(dev)), 1.0 + m1 @ m2)
        b1, b2 = torch.randn(6, 17, 32), torch.randn(6, 32, 9)
        assert close(torch.bmm(b1.to(dev), b2.to(dev)), torch.bmm(b1, b2))
        x4 = torch.randn(2, 3, 17, 32)
        assert close(torch.matmul(x4.to(dev), b2[:3].to(dev)), torch.matmul(x4, b2[:3]))
        lin = torch.nn.Linear(24, 56); x = torch.randn(5, 7, 24)
        with torch.no_grad():
            ref_lin = lin(x)
            assert close(lin.to(dev)(x.to(dev)), ref_lin)                                     # Module.to moves the parameters in place
        # the first benchmark configuration: Linear(64,128) -> ReLU -> Linear(128,10), batch 32, float32, seed 0
        torch.manual_seed(0)
        mlp = torch.nn.Sequential(torch.nn.Linear(64, 128), torch.nn.ReLU(), torch.nn.Linear(128, 10)).eval()
        xb = torch.randn(32, 64)
        with torch.no_grad():
            ref = mlp(xb)
            got = mlp.to(dev)(xb.to(dev))
        assert got.device.type == "applegpu" and close(got, ref)
        # embedding, layer_norm, softmax
        table = torch.randn(100, 48); ids = torch.randint(0, 100, (4, 9))
        assert torch.equal(F.embedding(ids.to(dev), table.to(dev)).cpu(), F.embedding(ids, table))
        g, be = torch.randn(48), torch.randn(48); y = torch.randn(4, 9, 48)
        assert close(F.layer_norm(y.to(dev), (48,), g.to(dev), be.to(dev), 1e-5), F.layer_norm(y, (48,), g, be, 1e-5), 1e-5)
        assert close(torch.softmax(y.to(dev), -1), torch.softmax(y, -1), 1e-5)
        assert close(torch.softmax(y.to(dev), 1), torch.softmax(y, 1), 1e-5)                 # not the last dim: CPU fallback
        launched = lib.applegpu_launch_count() - n0
        # fused attention behind scaled_dot_product_attention; a masked call decomposes into the ops above
        q, k, v = torch.randn(2, 4, 96, 64), torch.randn(2, 4, 96, 64), torch.randn(2, 4, 96, 64)
        n1 = lib.applegpu_launch_count()
        got = F.scaled_dot_product_attention(q.to(dev), k.to(dev), v.to(dev), is_causal=True)
        fused_launches = lib.applegpu_launch_count() - n1
        assert close(got, F.scaled_dot_product_attention(q, k, v, is_causal=True), 1e-4)
        assert fused_launches <= 2, fused_launches                                            # one attention kernel, no score matrix
        assert close(F.scaled_dot_product_attention(q.to(dev), k.to(dev), v.to(dev)), F.scaled_dot_product_attention(q, k, v), 1e-4)
        mask = torch.rand(96, 96) > 0.3; mask[:, 0] = True
        assert close(F.scaled_dot_product_attention(q.to(dev), k.to(dev), v.to(dev), attn_mask=mask.to(dev)), F.scaled_dot_product_attention(q, k, v, attn_mask=mask), 1e-4)
        q1 = torch.randn(2, 4, 1, 64)                                                         # a decode step against a longer cache
        assert close(F.scaled_dot_product_attention(q1.to(dev), k.to(dev), v.to(dev)), F.scaled_dot_product_attention(q1, k, v), 1e-4)
        # bf16 runs on the tensor-core path
        xb16, wb16 = torch.randn(256, 512).bfloat16(), torch.randn(512, 384).bfloat16()
        assert close(torch.mm(xb16.to(dev), wb16.to(dev)).float(), xb16.float() @ wb16.float(), 1e-2)
        # an op with no device kernel goes through the CPU fallback and comes back on the device
        s = torch.cumsum(ga, 1)
        assert s.device.type == "applegpu" and close(s, torch.cumsum(a, 1))
        assert ga.argmax().item() == a.argmax().item()
        print("ok", launched)
    """)
    assert out.strip().startswith("ok") and int(out.split()[1]) > 40


_GPT2 = """
    from transformers import GPT2Config, GPT2LMHeadModel
    torch.manual_seed(0)
    model = GPT2LMHeadModel(GPT2Config()).eval()           # GPT-2 small: 12 layers, 12 heads, 768 wide, 50257 tokens; seeded random weights
    prompt = [15496, 995]
"""


@pytest.mark.gpu
def test_hf_gpt2_greedy_generation_equals_cpu():
    """python/tests/test_cpp_backend.py:396-436: five greedy tokens, no cache, CPU == applegpu."""
    out = _run(_GPT2, """
        ids_cpu = list(prompt)
        with torch.no_grad():
            for _ in range(5):
                logits = model(torch.tensor([ids_cpu])).logits
                ids_cpu.append(logits[:, -1:].argmax(-1)[0, 0].item())
            last_cpu = model(torch.tensor([ids_cpu])).logits[0, -1]
        n0 = lib.applegpu_launch_count()
        model_gpu = model.to("applegpu").eval()
        assert next(model_gpu.parameters()).device.type == "applegpu"
        ids_gpu = list(prompt)
        with torch.no_grad():
            for _ in range(5):
                gen = torch.tensor([ids_gpu], device="applegpu")
                out = model_gpu(gen)
                assert out.logits.device.type == "applegpu"
                ids_gpu.append(out.logits[:, -1:].argmax(-1)[0, 0].cpu().item())
            last_gpu = model_gpu(torch.tensor([ids_gpu], device="applegpu")).logits[0, -1].cpu()
        assert ids_cpu == ids_gpu, (ids_cpu, ids_gpu)
        err = float((last_gpu - last_cpu).abs().max() / last_cpu.abs().max())
        assert err < 1e-4, err
        assert lib.applegpu_host_visible() == 0 and lib.applegpu_pipeline_status() == 0
        print("ok", lib.applegpu_launch_count() - n0, err)
    """)
    assert out.strip().startswith("ok") and int(out.split()[1]) > 6 * 12 * 8


@pytest.mark.gpu
def test_hf_gpt2_kv_cache_generation_equals_cpu():
    """python/tests/test_cpp_backend.py:439-480: prefill, then four single-token steps on the returned cache."""
    out = _run(_GPT2, """
        def generate(m, device):
            ids = list(prompt)
            with torch.no_grad():
                out = m(torch.tensor([ids], device=device), use_cache=True)
                past = out.past_key_values
                nt = out.logits[:, -1:].argmax(-1)
                ids.append(nt[0, 0].cpu().item())
                for _ in range(4):
                    out = m(nt, past_key_values=past, use_cache=True)
                    past = out.past_key_values
                    nt = out.logits[:, -1:].argmax(-1)
                    ids.append(nt[0, 0].cpu().item())
            return ids
        ids_cpu = generate(model, "cpu")
        ids_gpu = generate(model.to("applegpu").eval(), "applegpu")
        assert ids_cpu == ids_gpu, (ids_cpu, ids_gpu)
        print("ok")
    """)
    assert out.strip() == "ok"
