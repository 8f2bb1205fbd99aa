"""Host-runtime benchmarks (no GPU): the native token loader against a torch DataLoader over the
same file, the TCP transport's star / ring all-reduce on loopback, GGUF dequantisation, the
grammar mask walk (native against Python), the JSON-lines state-dict format and the host Philox
generator.

    python benchmarks/bench_host.py [--quick]

Prints one JSON line per measurement.
"""
import argparse
import json
import multiprocessing as mp
import os
import random
import socket
import string
import sys
import tempfile
import time

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def emit(name, **kw):
    print(json.dumps({"bench": name, **kw}), flush=True)


# --------------------------------------------------------------------------- token loader
class _WindowDataset(torch.utils.data.Dataset):
    def __init__(self, path, seq_len):
        self.a, self.s = np.memmap(path, dtype=np.uint16, mode="r"), seq_len

    def __len__(self):
        return (len(self.a) - 1) // self.s

    def __getitem__(self, i):
        w = torch.from_numpy(self.a[i * self.s:i * self.s + self.s + 1].astype(np.int64))
        return w[:-1], w[1:]


def bench_loader(quick):
    from ferrotorch_b200.data.token_loader import TokenFileLoader, write_token_file

    n_tokens, S, B = (8 << 20, 2048, 8) if quick else (64 << 20, 4096, 8)
    path = os.path.join(tempfile.mkdtemp(), "tokens.bin")
    write_token_file(path, torch.randint(0, 50000, (n_tokens,)), 50000)
    for workers in (1, 4):
        ld = TokenFileLoader(path, S, B, num_workers=workers, prefetch=8, seed=1, pin_memory=False)
        t0, n = time.perf_counter(), 0
        for x, _ in ld:
            n += x.numel()
        dt = time.perf_counter() - t0
        emit("token_loader_native", workers=workers, seq_len=S, batch=B, tokens_per_s=n / dt, gb_per_s_int64=n * 8 / dt / 1e9)
        ld.close()
    for workers in (0, 4):
        dl = torch.utils.data.DataLoader(_WindowDataset(path, S), batch_size=B, shuffle=True, num_workers=workers, drop_last=True)
        t0, n = time.perf_counter(), 0
        for x, _ in dl:
            n += x.numel()
        dt = time.perf_counter() - t0
        emit("token_loader_torch_dataloader", workers=workers, seq_len=S, batch=B, tokens_per_s=n / dt)


# --------------------------------------------------------------------------- TCP all-reduce
def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _ar_worker(rank, world, port, n, iters, q):
    from ferrotorch_b200.parallel.backend import TcpGroup

    g = TcpGroup(rank, world, "127.0.0.1", port, timeout=60.0)
    t = torch.ones(n)
    out = {}
    for algo in ("star", "ring"):
        g.all_reduce(t.clone(), "sum", algorithm=algo)          # connections, first touch
        g.barrier()
        t0 = time.perf_counter()
        for _ in range(iters):
            g.all_reduce(t, "mean", algorithm=algo)
        g.barrier()
        out[algo] = (time.perf_counter() - t0) / iters
    g.close()
    q.put((rank, out))


def bench_allreduce(quick):
    ctx = mp.get_context("spawn")
    for world in (2, 4):
        for n in ((1 << 20,) if quick else (1 << 16, 1 << 20, 1 << 24)):
            q, port = ctx.Queue(), _free_port()
            ps = [ctx.Process(target=_ar_worker, args=(r, world, port, n, 5 if n >= 1 << 24 else 20, q)) for r in range(world)]
            for p in ps:
                p.start()
            res = dict(q.get(timeout=300) for _ in range(world))
            for p in ps:
                p.join(30)
            for algo in ("star", "ring"):
                sec = max(r[algo] for r in res.values())
                emit("tcp_all_reduce_loopback", world=world, floats=n, algorithm=algo, ms=sec * 1e3,
                     algbw_gb_per_s=n * 4 / sec / 1e9)


# --------------------------------------------------------------------------- GGUF, grammar, state dict
def bench_gguf(quick):
    from ferrotorch_b200.serialize import gguf as G

    rows, cols = (2048, 4096) if quick else (8192, 8192)
    blocks = G.quantize_q4_0(torch.randn(rows, cols)).reshape(-1)
    for order in ("ggml", "interleaved"):
        t0 = time.perf_counter()
        G.dequantize_blocks(blocks, G.GGML_Q4_0, rows * cols, order)
        dt = time.perf_counter() - t0
        emit("gguf_q4_0_dequantize_host", elements=rows * cols, nibble_order=order, ms=dt * 1e3, gelem_per_s=rows * cols / dt / 1e9)


def bench_grammar(quick):
    from ferrotorch_b200.utils.grammar import JsonSchemaProcessor

    schema = {"type": "object", "properties": {"name": {"type": "string"}, "age": {"type": "integer", "minimum": 0, "maximum": 150},
                                                "tags": {"type": "array", "items": {"enum": ["a", "b", "c"]}}}, "required": ["name", "age"]}
    random.seed(0)
    n = 32000 if quick else 128000
    alphabet = string.ascii_letters + string.digits + ' {}[]":,.-_'
    vocab = ["<eos>"] + ["".join(random.choice(alphabet) for _ in range(random.randint(1, 6))) for _ in range(n)]
    for native in (True, False):
        t0 = time.perf_counter()
        p = JsonSchemaProcessor(schema, vocab, 0, native=native)
        build = time.perf_counter() - t0
        p.grammar().step_text('{"name":"ab')                       # inside an unbounded string: nearly every token is admitted
        t0 = time.perf_counter()
        m = p.compute_mask()
        cold = time.perf_counter() - t0
        p.grammar().step_text('c","age":1')
        t0 = time.perf_counter()
        p.compute_mask()
        other = time.perf_counter() - t0
        emit("grammar_token_mask", vocab=len(vocab), native=native, trie_build_s=build, mask_in_string_ms=cold * 1e3,
             mask_after_digit_ms=other * 1e3, admitted=m.num_allowed())


def bench_state_dict(quick):
    from ferrotorch_b200.serialize import state as S

    n = 8 if quick else 256
    sd = {"layer%d.weight" % i: torch.randn(1024, 1024) for i in range(n)}
    base = "/dev/shm" if os.path.isdir("/dev/shm") else None       # memory-backed: measures the code, not the disk
    path = os.path.join(tempfile.mkdtemp(dir=base), "m.ftsd")
    S.save_state_dict(sd, path)                                  # first write allocates the file's pages
    t0 = time.perf_counter()
    S.save_state_dict(sd, path)
    w = time.perf_counter() - t0
    mb = n * 4
    rates = {}
    for threads in (1, 4, 8):
        S.load_state_dict(path, threads=threads)
        t0 = time.perf_counter()
        S.load_state_dict(path, threads=threads)
        rates["read_mb_per_s_%d_threads" % threads] = mb / (time.perf_counter() - t0)
    t0 = time.perf_counter()
    lazy = S.load_state_dict(path, mmap=True)
    rates["mmap_open_ms"] = (time.perf_counter() - t0) * 1e3
    t0 = time.perf_counter()
    sum(float(v.sum()) for v in lazy.values())
    rates["mmap_first_touch_mb_per_s"] = mb / (time.perf_counter() - t0)
    del lazy
    t0 = time.perf_counter()
    buf = bytearray(os.path.getsize(path))
    with open(path, "rb") as f:
        f.readinto(buf)
    S.loads_state_dict(buf)
    rates["read_mb_per_s_single_readinto"] = mb / (time.perf_counter() - t0)
    emit("native_state_dict", megabytes=mb, write_mb_per_s=mb / w, filesystem=base or "tmp", **rates)
    try:
        from safetensors.torch import load_file, save_file

        st = path + ".safetensors"
        save_file(sd, st)
        load_file(st)
        t0 = time.perf_counter()
        load_file(st)
        emit("safetensors_library_load", megabytes=mb, read_mb_per_s=mb / (time.perf_counter() - t0))
        os.remove(st)
    except Exception:  # noqa: BLE001
        pass
    os.remove(path)


def bench_philox(quick):
    from ferrotorch_b200.utils.philox import PhiloxGenerator

    n = (1 << 20) if quick else (1 << 24)
    g = PhiloxGenerator(1)
    g.generate_uniform(1024)
    t0 = time.perf_counter()
    g.generate_uniform(n)
    u = time.perf_counter() - t0
    t0 = time.perf_counter()
    g.generate_normal(n)
    nrm = time.perf_counter() - t0
    emit("philox_host_generator", values=n, uniform_mvalues_per_s=n / u / 1e6, normal_mvalues_per_s=n / nrm / 1e6)


def bench_detection_ops(quick):
    """Greedy NMS and RoI align of the host library against their torch formulations."""
    import torch

    from ferrotorch_b200.ops import det_ops as D

    torch.manual_seed(0)
    n = 1000 if quick else 4000
    xy, wh = torch.rand(n, 2) * 500, torch.rand(n, 2) * 80 + 2
    boxes, scores = torch.cat([xy, xy + wh], 1), torch.rand(n)
    for name, fn in (("native", D.nms), ("torch", D.nms_torch)):
        fn(boxes, scores, 0.5)
        t0 = time.perf_counter()
        kept = fn(boxes, scores, 0.5)
        emit("nms_host", implementation=name, boxes=n, kept=len(kept), ms=(time.perf_counter() - t0) * 1e3)
    feat = torch.randn(2, 256, 50, 68)
    k = 128 if quick else 512
    rois = torch.cat([torch.randint(0, 2, (k, 1)).float(), boxes[:k] * 0.5], 1)
    for name, fn in (("native", D.roi_align), ("torch", D.roi_align_torch)):
        fn(feat, rois[:8], 7, 0.25, 2)
        t0 = time.perf_counter()
        fn(feat, rois, 7, 0.25, 2)
        emit("roi_align_host", implementation=name, rois=k, channels=256, ms=(time.perf_counter() - t0) * 1e3)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--quick", action="store_true")
    ap.add_argument("--only", default="")
    args = ap.parse_args()
    torch.set_num_threads(max(1, (os.cpu_count() or 2) // 2))
    benches = {"loader": bench_loader, "allreduce": bench_allreduce, "gguf": bench_gguf, "grammar": bench_grammar,
               "state_dict": bench_state_dict, "philox": bench_philox, "detection": bench_detection_ops}
    for name, fn in benches.items():
        if not args.only or name in args.only.split(","):
            fn(args.quick)


if __name__ == "__main__":
    main()
