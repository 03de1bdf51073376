"""Post-training int8 calibration: floating-point `.phai` / `.racy` in, int8 `.phai` / `.racy` out.

    python -m excalibur_b200.calibrate model.phai model.racy out.phai out.racy
           [--images N] [--size H W] [--range LO HI] [--percentile P] [--keep name1,name2] [--device 0]

The reference exposes the conv-input tensors to an external calibrator
(src/Excalibur/pipeline.cpp:271-277,639-652) and reads quantised convolutions from weight records
tagged 871224 (src/Excalibur/operation_convolution.cpp:115-145); this tool is that calibrator:

* runs the floating-point graph op by op on this library's pipeline over seeded random calibration
  images (uniform in --range; real calibration images can be passed by calling `convert()` from
  Python) and takes fs = 127 / max|x| (or 127 / the P-th percentile of |x|) of every dense
  convolution's input feature map;
* quantises the weights per output channel, ws[c] = 127 / max|w[c]|, wq = round(w * ws[c]);
* rewrites the conv's parameter line with key 8=1 and its weight record as int8 weights (padded to
  4 bytes), fp32 bias, ws[Cout], fs.

Depthwise / grouped convolutions, the first convolution of the graph, InnerProduct and every other
operation keep their floating-point records (names in --keep are left alone as well).
"""
import argparse
import struct

import numpy as np

from .modelfile import RACY_TAG_F32, RACY_TAG_I8


# ---- readers ------------------------------------------------------------------------------------
def parse_phai(text):
    """-> (header lines, [op dict(type, name, ins, outs, params {key: str}, order [keys])])."""
    lines = [l.rstrip() for l in text.splitlines() if l.strip()]
    head, body = lines[:2], lines[2:]
    ops = []
    for l in body:
        t = l.split()
        n_in, n_out = int(t[2]), int(t[3])
        ins, outs = t[4:4 + n_in], t[4 + n_in:4 + n_in + n_out]
        params, order = {}, []
        for kv in t[4 + n_in + n_out:]:
            k, v = kv.split("=", 1)
            params[int(k)] = v
            order.append(int(k))
        ops.append(dict(type=t[0], name=t[1], ins=ins, outs=outs, params=params, order=order))
    return head, ops


def op_line(op):
    toks = [op["type"], op["name"], str(len(op["ins"])), str(len(op["outs"]))] + op["ins"] + op["outs"]
    toks += ["%d=%s" % (k, op["params"][k]) for k in op["order"]]
    return " ".join(toks)


def racy_record_size(op, blob, pos):
    """Bytes the op's init_weights(FILE*) consumes at `pos` (file order = op order)."""
    t = op["type"].lower()
    p = op["params"]
    if t in ("convolution", "convolutiondepthwise", "deconvolution"):
        cout, wsize, bias = int(p[0]), int(p[6]), int(p.get(5, "0"))
        tag, = struct.unpack_from("<i", blob, pos)
        if tag == RACY_TAG_F32:
            return 4 + 4 * wsize + 4 * cout * bias
        if tag == RACY_TAG_I8:
            return 4 + (wsize + 3) // 4 * 4 + 4 * cout * bias + 4 * cout + 4
        raise ValueError("%s: unknown weight tag %d" % (op["name"], tag))
    if t == "innerproduct":
        nout, bias, wsize = int(p[0]), int(p.get(1, "0")), int(p[2])
        return 4 + 4 * wsize + 4 * nout * bias
    if t == "batchnorm":
        return 16 * int(p[0])
    if t == "prelu":
        return 4 * int(p[0])
    return 0


# ---- conversion ---------------------------------------------------------------------------------
def convert(phai_text, racy_bytes, images, percentile=None, keep=(), device=0):
    """Returns (int8 phai text, int8 racy bytes, {conv name: fs})."""
    from . import host
    head, ops = parse_phai(phai_text)
    # byte range of every op's record
    pos, spans = 0, []
    for op in ops:
        n = racy_record_size(op, racy_bytes, pos)
        spans.append((pos, n))
        pos += n
    if pos != len(racy_bytes):
        raise ValueError("weight file has %d bytes, the graph consumes %d" % (len(racy_bytes), pos))
    produced = set()
    for op in ops:
        produced.update(op["outs"])
    first_conv = next((op["name"] for op in ops if op["type"].lower() == "convolution"), None)
    targets = []
    for op, (p0, n) in zip(ops, spans):
        if op["type"].lower() != "convolution" or op["name"] in keep or op["name"] == first_conv:
            continue
        if int(op["params"].get(7, "1")) != 1 or int(op["params"].get(8, "0")) != 0:
            continue
        targets.append(op)
    pipe = host.Pipeline(phai_text, racy_bytes, device, fusion=False)
    pipe.forward(np.ascontiguousarray(images, np.float32))
    stats = {}
    for op in targets:
        fm = op["ins"][0]
        if fm not in stats:
            a = np.abs(pipe.get(fm))
            stats[fm] = float(a.max() if percentile is None else np.percentile(a, percentile))
    pipe.close()
    scales = {op["name"]: np.float32(127.0 / max(stats[op["ins"][0]], 1e-12)) for op in targets}
    out = bytearray()
    tnames = {op["name"] for op in targets}
    for op, (p0, n) in zip(ops, spans):
        if op["name"] not in tnames:
            out += racy_bytes[p0:p0 + n]
            continue
        prm = op["params"]
        cout, wsize, bias = int(prm[0]), int(prm[6]), int(prm.get(5, "0"))
        w = np.frombuffer(racy_bytes, "<f4", wsize, p0 + 4).reshape(cout, -1)
        b = np.frombuffer(racy_bytes, "<f4", cout, p0 + 4 + 4 * wsize) if bias else None
        ws = (127.0 / np.maximum(np.abs(w).max(axis=1), 1e-12)).astype(np.float32)
        wq = np.clip(np.rint(w * ws[:, None]), -127, 127).astype(np.int8)
        raw = wq.tobytes()
        raw += b"\0" * ((-len(raw)) % 4)
        out += struct.pack("<i", RACY_TAG_I8) + raw
        if b is not None:
            out += np.ascontiguousarray(b, "<f4").tobytes()
        out += ws.astype("<f4").tobytes() + struct.pack("<f", float(scales[op["name"]]))
        prm[8] = "1"
        if 8 not in op["order"]:
            op["order"].append(8)
    text = "\n".join(head + [op_line(op) for op in ops]) + "\n"
    return text, bytes(out), scales


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("phai")
    ap.add_argument("racy")
    ap.add_argument("out_phai")
    ap.add_argument("out_racy")
    ap.add_argument("--images", type=int, default=32)
    ap.add_argument("--size", type=int, nargs=2, default=[224, 224], metavar=("H", "W"))
    ap.add_argument("--channels", type=int, default=3)
    ap.add_argument("--range", type=float, nargs=2, default=[0.0, 1.0], metavar=("LO", "HI"))
    ap.add_argument("--percentile", type=float, default=None)
    ap.add_argument("--keep", default="")
    ap.add_argument("--seed", type=int, default=7)
    ap.add_argument("--device", type=int, default=0)
    args = ap.parse_args(argv)
    text = open(args.phai).read()
    blob = open(args.racy, "rb").read()
    x = np.random.default_rng(args.seed).uniform(args.range[0], args.range[1],
                                                 (args.images, args.channels, args.size[0], args.size[1]))
    t8, b8, scales = convert(text, blob, x.astype(np.float32), args.percentile,
                             tuple(k for k in args.keep.split(",") if k), args.device)
    open(args.out_phai, "w").write(t8)
    open(args.out_racy, "wb").write(b8)
    print("quantised %d convolutions; wrote %s (%d bytes) and %s (%d bytes)" % (
        len(scales), args.out_phai, len(t8), args.out_racy, len(b8)))


if __name__ == "__main__":
    main()
