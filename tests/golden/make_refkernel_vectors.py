"""Generates refkernel_vectors.npz: outputs of the reference engine's own CUDA kernels, rebuilt
for sm_100a from the reference sources (make -C oracle ref), on small seeded inputs.

Run on a machine with a B200 where oracle/_ref/libqwen_ref_{ieee,fastmath}.so exist:
    python tests/golden/make_refkernel_vectors.py [out.npz]
The file holds inputs and the reference's outputs for both builds ("ieee" = the sources as written,
"fastmath" = with the reference's own --use_fast_math flag), so the CPU oracle can be pinned to the
reference without a GPU afterwards (tests/test_oracle_refkernels.py).
"""
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
from qwen_engine_b200 import synth  # noqa: E402
from tests import util  # noqa: E402
from tests.util import RefKernels  # noqa: E402

out_path = Path(sys.argv[1] if len(sys.argv) > 1 else ROOT / "tests" / "golden" / "refkernel_vectors.npz")
data = {}
sp = util.stream_ptr()


def dev(a):
    return util.to_dev(a)


def q8_buffers(n):
    return (torch.empty(n, dtype=torch.int8, device="cuda"), torch.empty(n // 128, dtype=torch.float32, device="cuda"),
            torch.empty(n // 8, dtype=torch.int32, device="cuda"))


rng = np.random.Generator(np.random.Philox(key=0xC0FFEE))
x_q = rng.standard_normal(2048).astype(np.float32)
x_q[:128] = 0.0
x_q[128:256] *= 1e-4
x_q[256:384] *= 300.0
x_q[384:512] = np.round(x_q[384:512] * 4) / 4          # many exact ties after scaling
x_q = x_q.astype(np.float16)
data["quant_x"] = x_q

N, K = 64, 512
gw, gs = synth.packed_weights(21, "ref.g", N, K), synth.scales(21, "ref.g", N, K)
gx = synth.activations(21, "ref.g", K)
gres = synth.activations(22, "ref.res", N)
data.update(gemv_w=gw, gemv_s=gs, gemv_x=gx, gemv_res=gres)

N2, K2 = 48, 1536
ow, os_ = synth.packed_weights(23, "ref.o", N2, K2), synth.scales(23, "ref.o", N2, K2)
ox = synth.activations(23, "ref.o", K2)
data.update(gemv2_w=ow, gemv2_s=os_, gemv2_x=ox)

I_, H_ = 40, 512
sw, ss = synth.packed_weights(24, "ref.sw", 2 * I_, H_), synth.scales(24, "ref.sw", 2 * I_, H_)
data.update(swiglu_w=sw, swiglu_s=ss)

nq, nkv, hd, Kq = 2, 1, 64, 256   # q/k/v widths are multiples of the reference's 64-wide GEMM tile
qkv_w = [synth.packed_weights(25, f"ref.qkv{i}", n, Kq) for i, n in enumerate((nq * hd, nkv * hd, nkv * hd))]
qkv_s = [synth.scales(25, f"ref.qkv{i}", n, Kq) for i, n in enumerate((nq * hd, nkv * hd, nkv * hd))]
qkv_x = synth.activations(25, "ref.qkv", Kq)
for i in range(3):
    data[f"qkv_w{i}"], data[f"qkv_s{i}"] = qkv_w[i], qkv_s[i]
data["qkv_x"] = qkv_x
data["qkv_dims"] = np.array([nq, nkv, hd, Kq], dtype=np.int32)

M = 8
px = synth.activations(26, "ref.p", M, K)
pres = synth.activations(27, "ref.pres", M, N)
data.update(prefill_x=px, prefill_res=pres)
pxq = synth.activations(28, "ref.pq", M, Kq)
data["prefill_qkv_x"] = pxq

nx = (synth.activations(29, "ref.n", 1536).astype(np.float32) * 2.5).astype(np.float16)
ng = (1.0 + 0.1 * synth.activations(30, "ref.g", 1536).astype(np.float32)).astype(np.float16)
data.update(norm_x=nx, norm_gamma=ng)

for flavour in ("ieee", "fastmath"):
    ref = RefKernels(flavour)
    f = flavour
    # Q8_1 quantiser
    q8, sc, s8 = q8_buffers(x_q.size)
    ref.call("ref_quantize_fp16_to_q8_1", dev(x_q), q8, sc, s8, x_q.size, sp)
    torch.cuda.synchronize()
    data[f"{f}_quant_q8"], data[f"{f}_quant_scale"], data[f"{f}_quant_sum8"] = util.to_np(q8), util.to_np(sc), util.to_np(s8)
    # W4A8 GEMV (+residual), the uint4 kernel
    q8, sc, s8 = q8_buffers(K)
    ref.call("ref_quantize_fp16_to_q8_1", dev(gx), q8, sc, s8, K, sp)
    y = torch.empty(N, dtype=torch.float16, device="cuda")
    ref.call("ref_gemv_w4a8", dev(gw), dev(gs), q8, sc, s8, dev(gres), y, N, K, sp)
    torch.cuda.synchronize()
    data[f"{f}_gemv_q8"], data[f"{f}_gemv_xscale"], data[f"{f}_gemv_y"] = util.to_np(q8), util.to_np(sc), util.to_np(y)
    # fp16-input GEMV (standalone kernel)
    y2 = torch.empty(N2, dtype=torch.float16, device="cuda")
    ref.call("ref_gemv_w4a16", dev(ow), dev(os_), dev(ox), None, y2, N2, K2, sp)
    torch.cuda.synchronize()
    data[f"{f}_gemv2_y"] = util.to_np(y2)
    # SwiGLU, both entry points
    q8h, sch, s8h = q8_buffers(H_)
    ref.call("ref_quantize_fp16_to_q8_1", dev(gx[:H_].copy()), q8h, sch, s8h, H_, sp)
    ys = torch.empty(I_, dtype=torch.float16, device="cuda")
    ref.call("ref_gemv_dual_gate_up_swiglu_w4a8", dev(sw), dev(ss), q8h, sch, s8h, ys, H_, I_, sp)
    ys2 = torch.empty(I_, dtype=torch.float16, device="cuda")
    ref.call("ref_gemv_dual_gate_up_swiglu_w4a16", dev(sw), dev(ss), dev(gx[:H_].copy()), ys2, H_, I_, sp)
    torch.cuda.synchronize()
    data[f"{f}_swiglu_y_w4a8"], data[f"{f}_swiglu_y_w4a16"] = util.to_np(ys), util.to_np(ys2)
    # fused QKV
    q8q, scq, s8q = q8_buffers(Kq)
    ref.call("ref_quantize_fp16_to_q8_1", dev(qkv_x), q8q, scq, s8q, Kq, sp)
    d_w = [dev(w) for w in qkv_w]
    d_s = [dev(s) for s in qkv_s]
    outs = [torch.empty(n, dtype=torch.float16, device="cuda") for n in (nq * hd, nkv * hd, nkv * hd)]
    pod = RefKernels.QKVPod(d_w[0].data_ptr(), d_s[0].data_ptr(), outs[0].data_ptr(), d_w[1].data_ptr(),
                            d_s[1].data_ptr(), outs[1].data_ptr(), d_w[2].data_ptr(), d_s[2].data_ptr(),
                            outs[2].data_ptr())
    ref.call("ref_gemv_qkv_w4a8", pod, q8q, scq, s8q, sp, Kq, nq, nkv, hd)
    torch.cuda.synchronize()
    for i in range(3):
        data[f"{f}_qkv_y{i}"] = util.to_np(outs[i])
    # prefill GEMM (+residual), merged QKV, SwiGLU
    yp = torch.empty((M, N), dtype=torch.float16, device="cuda")
    ref.call("ref_gemm_prefill_w4a16", dev(gw), dev(gs), dev(px), dev(pres), yp, M, N, K, sp, 0)
    outs = [torch.empty((M, n), dtype=torch.float16, device="cuda") for n in (nq * hd, nkv * hd, nkv * hd)]
    pod = RefKernels.QKVPod(d_w[0].data_ptr(), d_s[0].data_ptr(), outs[0].data_ptr(), d_w[1].data_ptr(),
                            d_s[1].data_ptr(), outs[1].data_ptr(), d_w[2].data_ptr(), d_s[2].data_ptr(),
                            outs[2].data_ptr())
    ref.call("ref_gemm_prefill_qkv_w4a16", pod, dev(pxq), M, sp, Kq, nq, nkv, hd, 0)
    ypsw = torch.empty((M, I_), dtype=torch.float16, device="cuda")
    ref.call("ref_gemm_prefill_dual_gate_up_swiglu_w4a16", dev(sw), dev(ss), dev(px[:, :H_].copy()), ypsw, M, sp, H_, I_)
    torch.cuda.synchronize()
    data[f"{f}_prefill_y"] = util.to_np(yp)
    for i in range(3):
        data[f"{f}_prefill_qkv_y{i}"] = util.to_np(outs[i])
    data[f"{f}_prefill_swiglu_y"] = util.to_np(ypsw)
    # RMSNorm + Q8_1
    q8n, scn, s8n = q8_buffers(1536)
    yn = torch.empty(1536, dtype=torch.float16, device="cuda")
    ref.call("ref_rmsnorm_q8_1", dev(nx), dev(ng), yn, q8n, scn, s8n, sp, 1536)
    torch.cuda.synchronize()
    data[f"{f}_norm_y"], data[f"{f}_norm_q8"], data[f"{f}_norm_scale"] = util.to_np(yn), util.to_np(q8n), util.to_np(scn)

out_path.parent.mkdir(parents=True, exist_ok=True)
np.savez_compressed(out_path, **data)
print("wrote", out_path, len(data), "arrays")
