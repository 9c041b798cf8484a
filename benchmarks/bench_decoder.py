"""8-layer MoE decoder training step, expert-parallel over all GPUs of the node, timed against the
NCCL all-to-all baseline with no redundant experts (run under torch.distributed.run).

Defaults: hidden 2048, 16 heads, seq 4096 (micro-batch 1 per rank), 8 layers, 128 SwiGLU experts
with H'=768, top-8, vocab 32000, uniform random token ids with targets that are a fixed function of the token, router bias searched for MaxVio >= 4.

  python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 benchmarks/bench_decoder.py
"""
import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from moonep_b200.api import Buffer  # noqa: E402
from moonep_b200.models.decoder import MoEDecoder, NcclMoELayer  # noqa: E402
from moonep_b200.models.moe_layer import ExpertPools, MoELayer  # noqa: E402
from moonep_b200.ops import elementwise as ew  # noqa: E402
from moonep_b200.ops import gemm  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--hidden", type=int, default=2048)
    ap.add_argument("--heads", type=int, default=16)
    ap.add_argument("--seq", type=int, default=4096)
    ap.add_argument("--layers", type=int, default=8)
    ap.add_argument("--experts", type=int, default=128)
    ap.add_argument("--ffn", type=int, default=768)
    ap.add_argument("--topk", type=int, default=8)
    ap.add_argument("--vocab", type=int, default=32000)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--maxvio", type=float, default=4.0)
    ap.add_argument("--lr", type=float, default=1e-3)
    ap.add_argument("--impls", default="fused,nccl")
    ap.add_argument("--fused-sgd", action="store_true",
                    help="apply the expert weights' SGD step inside the weight-grad kernels (peer-memory path only)")
    ap.add_argument("--graph", action="store_true",
                    help="capture the fused step in a CUDA graph (off by default: with the dense-grad NCCL "
                         "all-reduce inside the graph, process-group teardown has been seen to stall)")
    args = ap.parse_args()
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    R, rank = dist.get_world_size(), dist.get_rank()
    S, Hd, E, K, Hp = args.seq, args.hidden, args.experts, args.topk, args.ffn
    gen = torch.Generator(device=dev).manual_seed(17 + rank)
    # Synthetic but LEARNABLE data: token ids are uniform random, the target of a position is a fixed
    # function of its token (an affine map modulo the vocabulary), so the loss falls from ln(vocab)
    # within the timed steps and a run shows that the stack trains, not only that it runs.
    def batch():
        tok = torch.randint(0, args.vocab, (S,), device=dev, generator=gen)
        return tok, (tok * 31 + 7) % args.vocab

    batches = [batch() for _ in range(4)]
    order = torch.randperm(E, generator=torch.Generator().manual_seed(99))
    ranks_ = torch.empty(E)
    ranks_[order] = torch.arange(1, E + 1, dtype=torch.float32)
    logpop = -torch.log(ranks_).to(dev)
    results = {}
    for impl in args.impls.split(","):
        torch.manual_seed(1234)                     # identical dense init on every rank / impl
        buf = pools = None
        if impl == "fused":
            buf = Buffer(S, Hd, K, E, R, num_sms=32 if R > 1 else 16, token_padding=128)
            pools = ExpertPools(R, E // R, Hd, Hp, buf.group, rank) if R > 1 else None
            factory = lambda i: MoELayer(buf, Hp, pools, seed=100 + i)
        else:
            factory = lambda i: NcclMoELayer(S, Hd, K, E, Hp, seed=100 + i)
        model = MoEDecoder(args.vocab, Hd, args.layers, args.heads, factory).to(dev)
        # router bias: Zipf popularity, exponent searched on the first block's router input
        with torch.no_grad():
            x0 = model.blocks[0].norm2(model.embed(batches[0][0]))
            logits = gemm.dense(x0.contiguous(), model.blocks[0].moe.w_router)
            lo, hi, best = 0.0, 8.0, (None, 1e9)
            for _ in range(18):
                mid = 0.5 * (lo + hi)
                b = (mid * logpop).contiguous()
                _, _, tpe = ew.router_topk(logits, K, b)
                tot = tpe.float()
                dist.all_reduce(tot)
                mv = float(tot.max() / tot.mean() - 1)
                if abs(mv - args.maxvio) < abs(best[1] - args.maxvio):
                    best = (b, mv)
                lo, hi = (mid, hi) if mv < args.maxvio else (lo, mid)
        for m in model.moe_layers():
            m.router_bias = best[0]
        torch.cuda.reset_peak_memory_stats(dev)
        losses = []
        for i in range(args.warmup):
            losses.append(float(model.train_step(*batches[i % 4], args.lr, args.fused_sgd)))
        # The fused path has static shapes and no host synchronisation, so the whole step
        # (~2400 launches for 8 layers) replays from one CUDA graph.  The NCCL baseline cannot:
        # its all_to_all split sizes are read back to the host every layer.
        run_step, graphed = (lambda tok, tgt: model.train_step(tok, tgt, args.lr, args.fused_sgd)), False
        if impl == "fused" and args.graph:
            try:
                from moonep_b200.utils.graph import GraphedStep
                gs = GraphedStep(lambda tok, tgt: model.train_step(tok, tgt, args.lr, args.fused_sgd), list(batches[0]), warmup=1)
                run_step, graphed = (lambda tok, tgt: gs(tok, tgt)), True
                float(run_step(*batches[1]))
            except Exception as exc:  # noqa: BLE001
                if rank == 0:
                    print(f"[bench_decoder] graph capture failed, eager: {type(exc).__name__}: {exc}",
                          file=sys.stderr, flush=True)
                run_step, graphed = (lambda tok, tgt: model.train_step(tok, tgt, args.lr, args.fused_sgd)), False
                torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        a, b2 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for i in range(args.steps):
            loss = run_step(*batches[i % 4])
        b2.record()
        torch.cuda.synchronize()
        ms = torch.tensor([a.elapsed_time(b2) / args.steps], device=dev)
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        peak = torch.tensor([torch.cuda.max_memory_allocated(dev) / 2 ** 30], device=dev)
        dist.all_reduce(peak, op=dist.ReduceOp.MAX)
        if buf is not None:
            buf.check()
        gemm.check_status(dev)
        results[impl] = {"ms_per_step": round(float(ms), 3), "tokens_per_s": round(R * S / float(ms) * 1e3, 1),
                         "peak_mem_gb_max_rank": round(float(peak), 2), "loss_first": losses[0],
                         "loss_last": float(loss), "maxvio_layer0": round(best[1], 3), "cuda_graph": graphed}
        del model
        if buf is not None:
            buf.destroy()
        torch.cuda.empty_cache()
    if rank == 0:
        out = {"bench": "moe_decoder_train", "n_gpus": R, "steps": args.steps,
               "config": {k: getattr(args, k) for k in ("hidden", "heads", "seq", "layers", "experts", "ffn", "topk", "vocab")},
               **results}
        if "fused" in results and "nccl" in results:
            out["speedup_vs_nccl"] = round(results["nccl"]["ms_per_step"] / results["fused"]["ms_per_step"], 3)
        print(json.dumps(out), flush=True)
    sys.stdout.flush()
    if args.graph:
        os._exit(0)          # see --graph: skip the collective teardown
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
