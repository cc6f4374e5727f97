"""Generate the golden fixtures of this folder by running the reference library's own Python
code on the CPU.  Needs a checkout of the reference; run as

    python tests/golden/make_golden.py /path/to/ads_model_kernel_library

The reference uses absolute imports ``ads_mkl.ops.oss.<package>``; a temporary directory with a
symlink of that name makes them resolve.  Four things are recorded:

* ``reference_cpu_softmax``: outputs of ``cpu_generalized_dot_product_attention``
  (gdpa/triton/triton_generalized_dot_product_attention.py:3898-3979) on a jagged batch with
  different Q and KV lengths;
* ``reference_eager_<activation>``: outputs of the eager helper ``_gdpa_reference``
  (gdpa_megakernel/tests/test_tlx_gdpa_megakernel.py:35-47), executed from the reference's file
  with the reference's activation table ``get_pytorch_activation`` (gdpa/triton/math.py:58-74);
  the helper's module cannot be imported whole because it needs a Triton fork, so the single
  function is taken from its source by ``ast`` and executed unchanged;
* ``triton_<activation>_{o,dq,dk,dv}``: outputs of the reference's Triton GDPA kernels themselves, the
  forward op body (gdpa/triton/triton_generalized_dot_product_attention.py:3099-3335) and the backward
  op body (:3461-3788), executed on the CPU by Triton's interpreter (``TRITON_INTERPRET=1``, autotuning
  off), on a jagged batch with different Q and KV lengths and ``qk_scale = 0.25``, for every activation
  of the table; plus one grouped-query case (4 query heads, 2 K/V heads), one banded case
  (``window_size = 6``), one case with per-head activations (``ensemble_activation_list``), one with
  ``broadcast_q`` and one with ``use_start_end_offsets`` (overlapping K / V ranges).  These pin where the scale is applied and every gradient;
* ``norms_{rms,ln_rms}_ref``: the expected values of the reference's two GDPA-plus-norm tests
  (gdpa_megakernel/tests/test_tlx_gdpa_megakernel.py:50-91 RMS norm after GDPA; :93-145 layer norm of Q, GDPA,
  Q residual, RMS norm), computed by the reference's own statements: the input generator
  ``_make_dense_jagged_inputs``, ``_gdpa_reference`` and the assignments to ``ln_q``, ``gdpa_ref`` and ``ref`` are
  taken from the test file by ``ast`` and executed unchanged on the CPU with the test's seed, shape and dtype
  (bf16; the kernel call itself needs a Triton fork and a GPU and is left out);
* ``activation_ids.json``: the reference's activation name -> id table (gdpa/triton/math.py:77-78).

Outputs: ``gdpa_golden.npz`` and ``activation_ids.json`` beside this script.
"""
from __future__ import annotations

import ast
import json
import os
import sys
import tempfile

# The Triton kernels of the reference run on the CPU through Triton's interpreter; both switches must be
# set before triton is imported.
os.environ.setdefault("TRITON_INTERPRET", "1")
os.environ.setdefault("GDPA_DISABLE_AUTOTUNE", "1")
os.environ.setdefault("ADS_MKL_DISABLE_AUTOTUNE", "1")

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def main(ref_root: str) -> None:
    shim = tempfile.mkdtemp(prefix="ads_mkl_shim_")
    os.makedirs(os.path.join(shim, "ads_mkl", "ops"))
    os.symlink(os.path.abspath(ref_root), os.path.join(shim, "ads_mkl", "ops", "oss"))
    sys.path.insert(0, shim)

    from ads_mkl.ops.oss.gdpa.triton import math as ref_math  # noqa: E402
    import ads_mkl.ops.oss.gdpa.triton.triton_generalized_dot_product_attention as ref_gdpa  # noqa: E402

    out = {}

    # ---- 1. the registered CPU kernel (softmax), Q and KV lengths differ -------------------
    rng = np.random.default_rng(1234)
    B, H, D = 5, 2, 16
    lq = rng.integers(1, 20, B)
    lk = rng.integers(1, 24, B)
    qo = torch.tensor(np.concatenate([[0], np.cumsum(lq)]), dtype=torch.int64)
    ko = torch.tensor(np.concatenate([[0], np.cumsum(lk)]), dtype=torch.int64)
    g = torch.Generator().manual_seed(1234)
    q = torch.randn(int(qo[-1]), H, D, generator=g)
    k = torch.randn(int(ko[-1]), H, D, generator=g)
    v = torch.randn(int(ko[-1]), H, D, generator=g)
    o = ref_gdpa.cpu_generalized_dot_product_attention(
        q, k, v, qo, ko, int(lq.max()), int(lk.max()), activation="raw"
    )
    out.update(
        softmax_q=q.numpy(), softmax_k=k.numpy(), softmax_v=v.numpy(),
        softmax_qo=qo.numpy(), softmax_ko=ko.numpy(), softmax_out=o.numpy(),
    )

    # ---- 2. the eager helper, every activation of the table --------------------------------
    src_path = os.path.join(ref_root, "gdpa_megakernel", "tests", "test_tlx_gdpa_megakernel.py")
    tree = ast.parse(open(src_path).read())
    fn = next(n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name == "_gdpa_reference")
    ns = {"torch": torch, "get_pytorch_activation": ref_math.get_pytorch_activation}
    exec(compile(ast.Module(body=[fn], type_ignores=[]), src_path, "exec"), ns)
    helper = ns["_gdpa_reference"]

    rng = np.random.default_rng(4321)
    B, H, D = 4, 2, 16
    ln = rng.integers(1, 24, B)
    off = torch.tensor(np.concatenate([[0], np.cumsum(ln)]), dtype=torch.int64)
    g = torch.Generator().manual_seed(4321)
    q = torch.randn(int(off[-1]), H, D, generator=g)
    k = torch.randn(int(off[-1]), H, D, generator=g)
    v = torch.randn(int(off[-1]), H, D, generator=g)
    out.update(eager_q=q.numpy(), eager_k=k.numpy(), eager_v=v.numpy(), eager_off=off.numpy())
    for act in ref_math.Activation:
        out[f"eager_out_{act.value}"] = helper(q, k, v, off, act).numpy()

    # ---- 3. the Triton forward and backward kernels under the interpreter --------------------
    from torch._library.custom_ops import OPDEFS

    fwd = OPDEFS["gdpa::generalized_dot_product_attention"]._init_fn
    bwd = OPDEFS["gdpa::generalized_dot_product_attention_backward"]._init_fn
    rng = np.random.default_rng(777)
    B, H, D = 3, 2, 16
    lq, lk = rng.integers(1, 40, B), rng.integers(1, 50, B)
    qo = torch.tensor(np.concatenate([[0], np.cumsum(lq)]), dtype=torch.int32)
    ko = torch.tensor(np.concatenate([[0], np.cumsum(lk)]), dtype=torch.int32)
    g = torch.Generator().manual_seed(777)
    q = torch.randn(int(qo[-1]), H, D, generator=g)
    k = torch.randn(int(ko[-1]), H, D, generator=g)
    v = torch.randn(int(ko[-1]), H, D, generator=g)
    do = torch.randn(int(qo[-1]), H, D, generator=g)
    scale = 0.25
    out.update(triton_q=q.numpy(), triton_k=k.numpy(), triton_v=v.numpy(), triton_do=do.numpy(),
               triton_qo=qo.numpy(), triton_ko=ko.numpy(), triton_scale=np.float32(scale))
    skipped = []
    for act in ref_math.Activation:
        try:
            o = fwd(q, k, v, qo, ko, int(lq.max()), int(lk.max()), qk_scale=scale, activation=act.value)
            res = bwd(do, q, k, v, o, qo, ko, B, H, 1, int(lq.max()), int(lk.max()), D, D, qk_scale=scale,
                      activation_enum_int=ref_math.activation_to_int[act])
        except Exception as e:  # activations written with inline PTX cannot run in the interpreter
            skipped.append(act.value)
            continue
        out[f"triton_{act.value}_o"] = o.numpy()
        out[f"triton_{act.value}_dq"] = res[0].numpy()
        out[f"triton_{act.value}_dk"] = res[1].numpy()
        out[f"triton_{act.value}_dv"] = res[2].numpy()
    # grouped-query attention: 4 query heads over 2 K/V heads (Q_GROUP = 2)
    Hq, G = 4, 2
    qg = torch.randn(int(qo[-1]), Hq, D, generator=g)
    kg = torch.randn(int(ko[-1]), Hq // G, D, generator=g)
    vg = torch.randn(int(ko[-1]), Hq // G, D, generator=g)
    dog = torch.randn(int(qo[-1]), Hq, D, generator=g)
    og = fwd(qg, kg, vg, qo, ko, int(lq.max()), int(lk.max()), qk_scale=scale, activation="gelu_approx")
    resg = bwd(dog, qg, kg, vg, og, qo, ko, B, Hq, G, int(lq.max()), int(lk.max()), D, D, qk_scale=scale,
               activation_enum_int=ref_math.activation_to_int[ref_math.Activation.GeLUApprox])
    out.update(gqa_q=qg.numpy(), gqa_k=kg.numpy(), gqa_v=vg.numpy(), gqa_do=dog.numpy(), gqa_o=og.numpy(),
               gqa_dq=resg[0].numpy(), gqa_dk=resg[1].numpy(), gqa_dv=resg[2].numpy())

    # banded attention: |q - kv| <= window_size
    W = 6
    ow = fwd(q, k, v, qo, ko, int(lq.max()), int(lk.max()), qk_scale=scale, window_size=W, activation="gelu_approx")
    resw = bwd(do, q, k, v, ow, qo, ko, B, H, 1, int(lq.max()), int(lk.max()), D, D, qk_scale=scale, window_size=W,
               activation_enum_int=ref_math.activation_to_int[ref_math.Activation.GeLUApprox])
    out.update(window_size=np.int32(W), window_o=ow.numpy(), window_dq=resw[0].numpy(), window_dk=resw[1].numpy(),
               window_dv=resw[2].numpy())

    # per-head activations: head 0 relu, head 1 leaky_relu (base activation raw)
    ens = [ref_math.activation_to_int[ref_math.Activation.ReLU], ref_math.activation_to_int[ref_math.Activation.LeakyReLU]]
    oe = fwd(q, k, v, qo, ko, int(lq.max()), int(lk.max()), qk_scale=scale, activation="raw", ensemble_activation_list=ens)
    rese = bwd(do, q, k, v, oe, qo, ko, B, H, 1, int(lq.max()), int(lk.max()), D, D, qk_scale=scale,
               activation_enum_int=0, ensemble_activation_list=ens)
    out.update(ensemble_ids=np.array(ens, dtype=np.int32), ensemble_o=oe.numpy(), ensemble_dq=rese[0].numpy(),
               ensemble_dk=rese[1].numpy(), ensemble_dv=rese[2].numpy())

    # broadcast_q: one Q sequence of 9 rows attended with by every KV sequence; output rows of batch element z
    # at output_offset[z]; dQ summed over the batch
    LB = 9
    qb = torch.randn(LB, H, D, generator=g)
    qob = torch.tensor([0, LB], dtype=torch.int32)
    oob = torch.arange(B + 1, dtype=torch.int32) * LB
    dob = torch.randn(B * LB, H, D, generator=g)
    ob = fwd(qb, k, v, qob, ko, LB, int(lk.max()), qk_scale=scale, output_offset=oob, broadcast_q=True,
             activation="gelu_approx")
    resb = bwd(dob, qb, k, v, ob, qob, ko, B, H, 1, LB, int(lk.max()), D, D, qk_scale=scale, output_offset=oob,
               broadcast_q=True, activation_enum_int=ref_math.activation_to_int[ref_math.Activation.GeLUApprox])
    out.update(bcast_q=qb.numpy(), bcast_do=dob.numpy(), bcast_o=ob.numpy(), bcast_dq=resb[0].float().numpy(),
               bcast_dk=resb[1].numpy(), bcast_dv=resb[2].numpy())

    # start / end offsets: [start_0, end_0, start_1, end_1, ...]; the Q ranges are disjoint (the second one leaves a
    # gap before the third), the K / V ranges overlap, so dK / dV sum over the sequences that read a row
    tq, tk = int(qo[-1]), int(ko[-1])
    q_pairs = torch.tensor([0, int(qo[1]), int(qo[1]), int(qo[2]) - 1, int(qo[2]), tq], dtype=torch.int32)
    k_pairs = torch.tensor([0, min(30, tk), min(10, tk), min(45, tk), min(20, tk), tk], dtype=torch.int32)
    mq = int((q_pairs[1::2] - q_pairs[0::2]).max())
    mk = int((k_pairs[1::2] - k_pairs[0::2]).max())
    ose = fwd(q, k, v, q_pairs, k_pairs, mq, mk, qk_scale=scale, use_start_end_offsets=True, total_num_objects=tq,
              activation="gelu_approx")
    rese = bwd(do, q, k, v, ose, q_pairs, k_pairs, B, H, 1, mq, mk, D, D, qk_scale=scale, use_start_end_offsets=True,
               activation_enum_int=ref_math.activation_to_int[ref_math.Activation.GeLUApprox])
    covered = torch.zeros(tq, dtype=torch.bool)
    for s0, e0 in zip(q_pairs[0::2].tolist(), q_pairs[1::2].tolist()):
        covered[s0:e0] = True
    ose[~covered] = 0  # rows no sequence owns are uninitialised memory in the reference's output (torch.empty, :3015)
    out.update(startend_q_pairs=q_pairs.numpy(), startend_k_pairs=k_pairs.numpy(), startend_o=ose.numpy(),
               startend_dq=rese[0].float().numpy(), startend_dk=rese[1].float().numpy(), startend_dv=rese[2].float().numpy())

    # ---- 4. the expected values of the reference's GDPA-plus-norm tests, by the tests' own statements ----------
    make_inputs = next(n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name == "_make_dense_jagged_inputs")
    cls = next(n for n in tree.body if isinstance(n, ast.ClassDef) and n.name == "TLXGDPAMegakernelTest")
    for method, tag in (("test_fused_rmsnorm_matches_reference", "rms"),
                        ("test_fused_layernorm_and_rmsnorm_matches_reference", "ln_rms")):
        body = next(n for n in cls.body if isinstance(n, ast.FunctionDef) and n.name == method).body
        wanted = {"dtype", "activation", "normalized_shape", "ln_q", "gdpa_ref", "ref"}
        stmts = [st for st in body if isinstance(st, ast.Assign) and len(st.targets) == 1
                 and isinstance(st.targets[0], ast.Name) and st.targets[0].id in wanted]
        seed = next(st for st in body if isinstance(st, ast.Expr) and "manual_seed" in ast.unparse(st))
        inputs = next(st for st in body if isinstance(st, ast.Assign) and "_make_dense_jagged_inputs" in ast.unparse(st))
        ns4 = {"torch": torch, "get_pytorch_activation": ref_math.get_pytorch_activation, "device": "cpu"}
        exec(compile(ast.Module(body=[make_inputs, fn], type_ignores=[]), src_path, "exec"), ns4)
        order = sorted([seed, inputs] + stmts, key=lambda st: st.lineno)
        exec(compile(ast.Module(body=order, type_ignores=[]), src_path, "exec"), ns4)
        assert ns4["dtype"] == torch.bfloat16 and ns4["q"].shape == (256, 2, 128)
        # bf16 values are stored as their 16 bits; both tests draw the same inputs (same seed, same calls)
        bits = lambda t: t.contiguous().view(torch.int16).numpy()
        for name in ("q", "k", "v"):
            if f"norms_{name}_bf16_bits" in out:
                assert np.array_equal(out[f"norms_{name}_bf16_bits"], bits(ns4[name]))
            out[f"norms_{name}_bf16_bits"] = bits(ns4[name])
        out[f"norms_{tag}_ref_bf16_bits"] = bits(ns4["ref"])
        out["norms_offsets"] = ns4["offsets"].numpy()

    np.savez_compressed(os.path.join(HERE, "gdpa_golden.npz"), **out)
    ids = {a.value: i for a, i in ref_math.activation_to_int.items()}
    with open(os.path.join(HERE, "activation_ids.json"), "w") as f:
        json.dump(ids, f, indent=1)
    print("wrote", len(out), "arrays;", ids)
    print("activations the Triton interpreter could not run (inline PTX):", skipped)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: make_golden.py /path/to/ads_model_kernel_library")
    main(sys.argv[1])
