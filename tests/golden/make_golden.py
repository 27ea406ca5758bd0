"""Generates the golden fixtures of this folder from the UNMODIFIED reference.

Needs the reference built into oracle/_ref (oracle/build_ref.sh), so it only runs where the
reference tree is mounted; the JSON files it writes are committed and are what the tests read on
machines that do not have the reference.

    python tests/golden/make_golden.py small      # tests/golden/small_cases.json   (~1 min)
    python tests/golden/make_golden.py configs    # tests/golden/configs.json       (~15 min)
    python tests/golden/make_golden.py cnn        # tests/golden/cnn_steps.json     (~10 min)
    python tests/golden/make_golden.py mm16k      # tests/golden/mm16k.json         (~10 min)
    python tests/golden/make_golden.py mm16k_reference   # the same file from the reference alone (~35 min)
    python tests/golden/make_golden.py optim      # tests/golden/optim_steps.json   (seconds)

Every value is produced by the reference's own CPU backend (repdl.backend.cpu, plus the exp2d /
log1d shim and repdl/ops.py's ATen div / sqrt).  The full 16384^3 product is first hashed from the
C oracle (`mm16k`, with 512 rows compared with the reference) and then recomputed entirely by the
reference's transB path (`mm16k_reference`), which replaces the hashes by the reference's own.
"""
import hashlib
import json
import os
import sys
import time

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(HERE))

import oracle  # noqa: E402
from cases import RefAdapter, build_cases, run_case, sha  # noqa: E402
from repdl_b200 import workloads  # noqa: E402


def dump(name, obj):
    path = os.path.join(HERE, name)
    with open(path, "w") as f:
        json.dump(obj, f, indent=1, sort_keys=True)
    print("wrote", path)


def meta():
    import platform
    return {"torch": torch.__version__, "glibc": platform.libc_ver()[1],
            "generated_from": "microsoft/RepDL CPU backend (backend/cpu/*.cpp), unmodified"}


def small(ref):
    impl = RefAdapter(ref)
    out = {"_meta": meta()}
    for case in build_cases():
        r = run_case(impl, case)
        out[case[0]] = {"sha256": sha(r), "shape": list(r.shape)}
    # a few raw values for eyeballing a failure
    from cases import special_values
    x = special_values(0)
    out["_specials_hex"] = {
        "x": [("%08x" % (v & 0xFFFFFFFF)) for v in x.view(torch.int32).tolist()],
        "exp": [("%08x" % (v & 0xFFFFFFFF)) for v in impl.exp(x).view(torch.int32).tolist()],
        "log": [("%08x" % (v & 0xFFFFFFFF)) for v in impl.log(x).view(torch.int32).tolist()],
        "sqrt": [("%08x" % (v & 0xFFFFFFFF)) for v in impl.sqrt(x).view(torch.int32).tolist()],
        "div10": [("%08x" % (v & 0xFFFFFFFF)) for v in impl.div(x, 10.0).view(torch.int32).tolist()],
    }
    dump("small_cases.json", out)


def configs(ref):
    impl = RefAdapter(ref)
    out = {"_meta": meta()}
    # config 1
    a, b = workloads.mm_square(1024, 0)
    t = time.time()
    out["c1_mm_1024"] = {"sha256": sha(impl.mm(a, b)), "input_sha256": [sha(a), sha(b)],
                         "ref_seconds": time.time() - t}
    # config 2: per-chunk and whole-array hashes of the four ops
    hs = {k: hashlib.sha256() for k in ("x", "div10", "sqrt_abs", "exp", "log_abs")}
    chunks = []
    for ci, x in enumerate(workloads.crmath_chunks(1 << 28, 1)):
        res = {"x": x, "div10": impl.div(x, 10.0), "sqrt_abs": impl.sqrt(x.abs()),
               "exp": impl.exp(x), "log_abs": impl.log(x.abs())}
        for k, v in res.items():
            hs[k].update(v.numpy().tobytes())
        chunks.append({k: sha(v) for k, v in res.items()})
        print("c2 chunk", ci, flush=True)
    out["c2_crmath_2p28"] = {"whole": {k: h.hexdigest() for k, h in hs.items()}, "chunks": chunks}
    # config 3: 1-D chain over 2^30 with the running state after every 2^24 chunk, and row sums
    state = torch.zeros(())
    states = []
    hx = hashlib.sha256()
    rows_h = hashlib.sha256()
    for ci, x in enumerate(workloads.sum_chunks(1 << 30, 2)):
        # reference sum1d starts at +0; carry the state by prepending it (0 + s == s exactly,
        # and for ci == 0 the state is +0)
        state = impl.sum1d(torch.cat([state.view(1), x]), False)
        states.append("%08x" % (state.view(torch.int32).item() & 0xFFFFFFFF))
        hx.update(x.numpy().tobytes())
        if ci < 16:
            rows_h.update(impl.sum2d_dim1(x.view(4096, 4096), False, False).numpy().tobytes())
        print("c3 chunk", ci, states[-1], flush=True)
    out["c3_sum1d_2p30"] = {"result_hex": states[-1], "state_after_chunk_hex": states,
                            "input_sha256": hx.hexdigest()}
    out["c3_sum_rows_65536x4096"] = {"sha256": rows_h.hexdigest()}
    dump("configs.json", out)


def cnn(ref):
    """Config 4 through the reference's own Python layers on its CPU backend."""
    sys.path.insert(0, ref.site)
    import repdl
    torch.manual_seed(3)
    model = repdl.from_torch_module(workloads.cnn_torch_model())
    x, y = workloads.cnn_batch(256)
    loss_fn = repdl.nn.CrossEntropyLoss()
    out = {"_meta": meta(), "init_params": repdl.utils.get_hash(model), "steps": []}
    out["input_sha256"] = [sha(x), sha(y)]
    for step in range(100):
        t = time.time()
        for p in model.parameters():
            p.grad = None
        logits = model(x)
        loss = loss_fn(logits, y)
        loss.backward()
        with torch.no_grad():
            for p in model.parameters():
                p.add_(p.grad.mul(-0.01))  # two roundings: the product, then the sum
        if step < 3 or step % 10 == 9:
            out["steps"].append({"step": step, "loss_hex": "%08x" % (loss.detach().view(torch.int32).item() & 0xFFFFFFFF),
                                 "logits": sha(logits), "params": repdl.utils.get_hash(model)})
        print("cnn step", step, float(loss), "%.1fs" % (time.time() - t), flush=True)
    with torch.no_grad():
        out["final_logits"] = sha(model(x))
    out["final_params"] = repdl.utils.get_hash(model)
    dump("cnn_steps.json", out)


def mm16k(ref):
    a, b = workloads.mm_large(16384, 4)
    out = {"_meta": meta(), "input_sha256": [sha(a), sha(b)]}
    t = time.time()
    c = oracle.mm(a, b)
    out["oracle_seconds"] = time.time() - t
    out["sha256"] = sha(c)
    # per-row-block hashes let a sharded run be checked shard by shard
    out["row_block_2048_sha256"] = [sha(c[i:i + 2048]) for i in range(0, 16384, 2048)]
    # pin against the reference on 512 rows spread over the matrix (its transB path on a
    # pre-transposed B gives the same chains, backend/cpu/matrix_multiplication.cpp:29-31)
    bt = b.t().contiguous()
    rows = torch.cat([torch.arange(s, s + 64) for s in range(0, 16384, 2048)])
    t = time.time()
    cr = ref.cpu.mm(a[rows].contiguous(), bt, False, True)
    out["reference_rows_checked"] = int(rows.numel())
    out["reference_rows_equal"] = bool(torch.equal(cr.view(torch.int32), c[rows].view(torch.int32)))
    out["reference_rows_seconds"] = time.time() - t
    assert out["reference_rows_equal"]
    dump("mm16k.json", out)


def mm16k_reference(ref):
    """Config 5 computed ENTIRELY by the reference's CPU backend (its transB path on a pre-transposed
    B: the same chains as the plain layout, backend/cpu/matrix_multiplication.cpp:29-31, at a
    cache-friendly stride), in row blocks, about half an hour on 8 cores.  Replaces the hashes of
    mm16k.json by the reference's own and records that they equal the C oracle's."""
    import hashlib
    path = os.path.join(HERE, "mm16k.json")
    out = json.load(open(path))
    a, b = workloads.mm_large(16384, 4)
    assert [sha(a), sha(b)] == out["input_sha256"]
    bt = b.t().contiguous()
    whole, blocks = hashlib.sha256(), []
    t = time.time()
    for r0 in range(0, 16384, 2048):
        blk = hashlib.sha256()
        for s0 in range(r0, r0 + 2048, 256):
            c = ref.cpu.mm(a[s0:s0 + 256].contiguous(), bt, False, True)
            raw = c.numpy().tobytes()
            whole.update(raw)
            blk.update(raw)
        blocks.append(blk.hexdigest())
        print("mm16k reference rows", r0 + 2048, "%.0fs" % (time.time() - t), flush=True)
    out["reference_full_seconds"] = time.time() - t
    out["reference_rows_checked"] = 16384
    out["reference_rows_equal"] = whole.hexdigest() == out["sha256"] and blocks == out["row_block_2048_sha256"]
    out["sha256_source"] = "reference CPU backend, whole product; equal to the C oracle's"
    assert out["reference_rows_equal"], (whole.hexdigest(), out["sha256"])
    out["sha256"], out["row_block_2048_sha256"] = whole.hexdigest(), blocks
    out.pop("reference_rows_seconds", None)
    dump("mm16k.json", out)


def optim(ref):
    """Parameter hashes after each of six steps of the reference's own Adam (repdl/optim.py) on CPU
    tensors, for four settings; and of the two-rounding SGD update written with torch's CPU ops."""
    import cases
    sys.path.insert(0, oracle.ref_site())
    import repdl
    out = {"_meta": meta()}
    for name, wd, ams in cases.OPTIM_CONFIGS:
        out["adam_" + name] = cases.run_optimizer(
            lambda ps: repdl.optim.Adam(ps, lr=0.01, weight_decay=wd, amsgrad=ams))

    class TwoRoundingSGD(torch.optim.Optimizer):
        def __init__(self, params, lr):
            super().__init__(params, dict(lr=lr))

        @torch.no_grad()
        def step(self):
            for group in self.param_groups:
                for p in group["params"]:
                    p.add_(p.grad.mul(-group["lr"]))
    out["sgd"] = cases.run_optimizer(lambda ps: TwoRoundingSGD(ps, 0.01))
    dump("optim_steps.json", out)


if __name__ == "__main__":
    ref = oracle.ref()
    if ref is None:
        sys.exit("oracle/_ref is not built (run oracle/build_ref.sh where the reference is mounted)")
    what = sys.argv[1:] or ["small"]
    for w in what:
        {"small": small, "configs": configs, "cnn": cnn, "mm16k": mm16k, "mm16k_reference": mm16k_reference,
         "optim": optim}[w](ref)
