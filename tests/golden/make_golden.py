"""Regenerates the golden fixtures of this directory.  Needs the EDDL source tree
(the directory ``$EDDL_REFERENCE`` names, or a checkout called ``reference`` beside this repository) and the reference CPU build
(``python oracle/build_ref.py cpu``); the fixtures themselves are committed so that the tests run
where neither is present.

reference_kats.json  numeric known-answer vectors read out of the reference's own unit tests
                     (tests/layers/conv/test_conv2d.cpp:9-393, tests/layers/pool/test_mpool.cpp:9-271,
                     tests/layers/pool/test_avgpool.cpp:8-272, tests/layers/conv/test_convol_sizes.cpp:10-41,
                     tests/losses/test_losses.cpp:18-40, tests/tensor/nn/test_tensor_nn.cpp:13-33).
ref_outputs.npz      outputs of the reference's own CPU code on seeded inputs for the parts its unit
                     tests do not pin: conv backward-weight, BatchNorm forward/backward, dense algebra,
                     SGD / Adam steps, Net::sync_weights arithmetic, and a 10-step loss/parameter
                     trajectory of the small CNN trained with eddl::train_batch on CS_CPU.
"""
import json
import os
import re
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
REF = os.environ.get("EDDL_REFERENCE") or os.path.join(os.path.dirname(ROOT), "reference")
sys.path.insert(0, ROOT)


def _eval_count(expr):
    return int(eval(expr.replace(" ", ""), {"__builtins__": {}}))


def _floats(body):
    body = re.sub(r"//[^\n]*", " ", body)
    return [float(t.rstrip("f")) for t in re.findall(r"[-+]?(?:\d+\.\d*|\.\d+|\d+)(?:[eE][-+]?\d+)?f?", body)]


def _test_blocks(path):
    text = open(path).read()
    heads = list(re.finditer(r"TEST\(\s*(\w+)\s*,\s*(\w+)\s*\)", text))
    for i, m in enumerate(heads):
        end = heads[i + 1].start() if i + 1 < len(heads) else len(text)
        yield m.group(2), text[m.end():end]


def _arrays(block):
    out = {}
    for m in re.finditer(r"auto\s*\*\s*(\w+)\s*=\s*new float\[([^\]]+)\]\s*\{(.*?)\};", block, flags=re.S):
        out[m.group(1)] = _floats(m.group(3))
    shapes = {}
    for m in re.finditer(r"new Tensor\(\{([\d,\s]+)\},\s*(\w+),\s*DEV_CPU\)", block):
        shapes[m.group(2)] = [int(v) for v in m.group(1).split(",")]
    return out, shapes


def conv_pool_kats(path, kind):
    cases = []
    for name, block in _test_blocks(path):
        if "cpu_gpu" in name or "3d" in name.lower():
            continue
        arrays, shapes = _arrays(block)
        if "ptr_img" not in arrays:
            continue
        case = {"name": name, "x": arrays["ptr_img"], "x_shape": shapes["ptr_img"],
                "fwd": arrays["ptr_fwrd"], "fwd_shape": shapes["ptr_fwrd"],
                "bwd": arrays["ptr_bwrd"], "bwd_shape": shapes["ptr_bwrd"]}
        if kind == "conv":
            m = re.search(r"new ConvolDescriptor\((\d+),\s*\{(\d+),\s*(\d+)\},\s*\{(\d+),\s*(\d+)\},\s*\"(\w+)\"", block)
            case.update(filters=int(m.group(1)), kernel=[int(m.group(2)), int(m.group(3))],
                        stride=[int(m.group(4)), int(m.group(5))], padding=m.group(6))
            if "ptr_kernels" in arrays:
                case["w"] = arrays["ptr_kernels"]; case["bias"] = arrays["ptr_bias"]
            else:     # Tensor::ones kernels, zero bias
                case["w"] = None; case["bias"] = None
        else:
            m = re.search(r"new PoolDescriptor\(\{(\d+),\s*(\d+)\},\s*\{(\d+),\s*(\d+)\},\s*\"(\w+)\"", block)
            case.update(kernel=[int(m.group(1)), int(m.group(2))], stride=[int(m.group(3)), int(m.group(4))], padding=m.group(5))
        cases.append(case)
    return cases


def size_table(path):
    text = open(path).read()
    m = re.search(r"output_sizes\s*=\s*\{(.*?)\};", text, flags=re.S)
    vals = [int(v) for v in _floats(m.group(1))]
    return {"padding": ["valid", "same"], "input_sizes": [3, 5, 8, 10], "strides": [1, 2, 3], "kernels": [1, 2, 3],
            "output_sizes": vals}


def small_kats():
    t = open(os.path.join(REF, "tests/losses/test_losses.cpp")).read()
    blk = t[t.index("losses_categorical_cross_entropy"):]
    tens = re.findall(r"new Tensor\(\{(.*?)\},\s*\{2,\s*3\}\)", blk, flags=re.S)[:3]
    cce = {"y_pred": _floats(tens[0]), "y_true": _floats(tens[1]), "delta_times_batch": _floats(tens[2]),
           "value_per_sample": float(re.search(r"ASSERT_NEAR\(value,\s*([\d.]+)f", blk).group(1)), "shape": [2, 3]}
    t = open(os.path.join(REF, "tests/tensor/nn/test_tensor_nn.cpp")).read()
    blk = t[t.index("tensor_nn_full_softmax"):]
    tens = re.findall(r"new Tensor\(\{(.*?)\},\s*\{2,\s*3\},\s*DEV_CPU\)", blk, flags=re.S)[:4]
    sm = {"x": _floats(tens[0]), "y": _floats(tens[1]), "delta": _floats(tens[2]), "parent_delta": _floats(tens[3]), "shape": [2, 3]}
    return cce, sm


def make_kats():
    cce, sm = small_kats()
    data = {
        "source": "EDDL v1.1 unit tests (numeric vectors only)",
        "tolerance": {"atol": 1e-3, "rtol": 0.0},
        "conv2d": conv_pool_kats(os.path.join(REF, "tests/layers/conv/test_conv2d.cpp"), "conv"),
        "maxpool2d": conv_pool_kats(os.path.join(REF, "tests/layers/pool/test_mpool.cpp"), "pool"),
        "avgpool2d": conv_pool_kats(os.path.join(REF, "tests/layers/pool/test_avgpool.cpp"), "pool"),
        "conv_output_sizes": size_table(os.path.join(REF, "tests/layers/conv/test_convol_sizes.cpp")),
        "cce": cce, "softmax": sm,
    }
    with open(os.path.join(HERE, "reference_kats.json"), "w") as f:
        json.dump(data, f)
    print("conv %d, maxpool %d, avgpool %d cases" % (len(data["conv2d"]), len(data["maxpool2d"]), len(data["avgpool2d"])))


def make_ref_outputs():
    from oracle import ref
    from eddl_b200 import harness
    rng = np.random.default_rng(20240607)
    out = {}
    # conv fwd / bwd-weight / bwd-data, stride 1 and 2, with and without bias
    for tag, (n, c, h, w, k, kr, st, pads, use_bias) in {
        "conv_a": (2, 3, 9, 8, 5, 3, 1, (1, 1, 1, 1), True),
        "conv_b": (3, 4, 11, 11, 6, 3, 2, (1, 1, 1, 1), False),
        "conv_c": (2, 8, 6, 6, 7, 1, 1, (0, 0, 0, 0), False),
        "conv_d": (2, 3, 14, 14, 4, 7, 2, (3, 3, 3, 3), False),
    }.items():
        x = rng.standard_normal((n, c, h, w)).astype(np.float32); wt = rng.standard_normal((k, c, kr, kr)).astype(np.float32)
        b = rng.standard_normal(k).astype(np.float32) if use_bias else None
        y, _, _, _ = ref.conv2d(x, wt, b, stride=(st, st), pads=pads)
        dy = rng.standard_normal(y.shape).astype(np.float32)
        gw0 = rng.standard_normal(wt.shape).astype(np.float32); dx0 = rng.standard_normal(x.shape).astype(np.float32)
        gb0 = rng.standard_normal(k).astype(np.float32) if use_bias else None
        y, gw, gb, dx = ref.conv2d(x, wt, b, dy, gw0, gb0, dx0, stride=(st, st), pads=pads)
        out.update({tag + "_x": x, tag + "_w": wt, tag + "_dy": dy, tag + "_gw0": gw0, tag + "_dx0": dx0, tag + "_y": y,
                    tag + "_gw": gw, tag + "_dx": dx, tag + "_meta": np.array([st, *pads, int(use_bias)])})
        if use_bias:
            out.update({tag + "_b": b, tag + "_gb0": gb0, tag + "_gb": gb})
    # batch norm (single OpenMP thread semantics do not matter for these sizes: <= 256 items per channel block)
    for tag, shape, affine, mom in (("bn_a", (4, 6, 5, 4), True, 0.99), ("bn_b", (8, 3, 7, 7), False, 0.9), ("bn_c", (16, 10), True, 0.0)):
        x = (rng.standard_normal(shape) * 2 + 0.5).astype(np.float32); z = shape[1]
        g = rng.standard_normal(z).astype(np.float32) if affine else None
        b = rng.standard_normal(z).astype(np.float32) if affine else None
        gm = rng.standard_normal(z).astype(np.float32); gv = rng.random(z).astype(np.float32) + 0.5
        f = ref.bn_fwd(x, gm, gv, g, b, True, 1e-3, mom)
        fe = ref.bn_fwd(x, f["gmean"], f["gvar"], g, b, False, 1e-3, mom)
        d = rng.standard_normal(shape).astype(np.float32); pd0 = rng.standard_normal(shape).astype(np.float32)
        gg0 = rng.standard_normal(z).astype(np.float32); gb0 = rng.standard_normal(z).astype(np.float32)
        opa = f["opa"] if affine else f["y"]
        bw = ref.bn_bwd(d, opa, pd0, gg0, gb0, g, f["var"])
        out.update({tag + "_x": x, tag + "_gm": gm, tag + "_gv": gv, tag + "_d": d, tag + "_pd0": pd0, tag + "_gg0": gg0, tag + "_gb0": gb0,
                    tag + "_y": f["y"], tag + "_mean": f["mean"], tag + "_var": f["var"], tag + "_gm1": f["gmean"], tag + "_gv1": f["gvar"],
                    tag + "_yeval": fe["y"], tag + "_vareval": fe["var"], tag + "_pd": bw["pdelta"], tag + "_dout": bw["delta"],
                    tag + "_m1": bw["m1"], tag + "_m2": bw["m2"]})
        if affine:
            out.update({tag + "_g": g, tag + "_b": b, tag + "_opa": f["opa"], tag + "_gg": bw["gg"], tag + "_gb": bw["gb"]})
    # dense algebra
    a = rng.standard_normal((7, 13)).astype(np.float32); bm = rng.standard_normal((13, 5)).astype(np.float32)
    c0 = rng.standard_normal((7, 5)).astype(np.float32)
    out.update(mm_a=a, mm_b=bm, mm_c0=c0, mm_nn=ref.mult2d(a, 0, bm, 0), mm_nn_inc=ref.mult2d(a, 0, bm, 0, c0, 1),
               mm_tn=ref.mult2d(a.T.copy(), 1, bm, 0), mm_nt=ref.mult2d(a, 0, bm.T.copy(), 1),
               rs_axis0=ref.reduce_sum2d(a, 0), rs_axis1=ref.reduce_sum2d(a, 1), rowbias=ref.sum2d_rowwise(a, a[0]))
    # optimizers
    p = rng.standard_normal(1000).astype(np.float32); g = rng.standard_normal(1000).astype(np.float32)
    m = rng.standard_normal(1000).astype(np.float32) * 0.1; v = rng.random(1000).astype(np.float32) * 0.01
    p1, m1 = ref.sgd_step(p, g, m, 0.1, 0.9)
    ap, ag, am, av = ref.adam_step(p, g, m, v, 0.01, 0.9, 0.999, 1e-6, 3)
    out.update(opt_p=p, opt_g=g, opt_m=m, opt_v=v, sgd_p=p1, sgd_m=m1, adam_p=ap, adam_g=ag, adam_m=am, adam_v=av)
    reps = rng.standard_normal((4, 513)).astype(np.float32)
    out.update(sync_reps=reps, sync_avg=ref.sync_weights(reps))
    # small-CNN trajectory on CS_CPU (threads=1 for a reproducible order)
    net = harness.NetHarness(ref.lib(), "cnn", device=-1, threads=1, optimizer="sgd", lr=0.01, mu=0.9)
    w0 = harness.init_weights(net.param_info(), seed=1234)
    net.set_params(w0)
    drng = np.random.default_rng(1234)
    x = drng.random((100, 1, 28, 28), dtype=np.float32); lab = drng.integers(0, 10, 100); y = np.eye(10, dtype=np.float32)[lab]
    losses = [net.train_batch(x, y)[0]]
    p1 = net.get_params()
    losses += [net.train_batch(x, y)[0] for _ in range(9)]
    out.update(cnn_losses=np.array(losses, np.float32), cnn_params_step1=p1, cnn_params_after=net.get_params(), cnn_labels=lab.astype(np.int32))
    net.close()
    np.savez_compressed(os.path.join(HERE, "ref_outputs.npz"), **out)
    print("ref_outputs.npz: %d arrays, cnn losses %s" % (len(out), np.array2string(np.array(losses[:4]), precision=6)))


if __name__ == "__main__":
    make_kats()
    make_ref_outputs()
