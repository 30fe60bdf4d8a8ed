"""Worker processes for the tensor-parallel tests (spawned by test_tp_*.py; not collected)."""
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)

from oracle import qwen_text, synth, tp as tp_oracle  # noqa: E402


def cpu_rank(rank, world, port, cfg_kw, seed, n_prompt, steps, out_dir):
    """gloo rank: tensor-parallel oracle vs nothing (rank 0 writes its logits / ids)."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(2)
    cfg = synth.tiny_config(**cfg_kw)
    w = synth.make_weights(cfg, seed=seed)
    prompt = synth.make_token_ids(n_prompt, seed=seed, vocab=cfg.vocab)
    o = tp_oracle.TpOracle(cfg, w, rank, world, "exact_fp32")
    logits, toks = [], []
    lg = o.forward(prompt)
    n_l = cfg.vocab // world
    for s in range(steps):
        logits.append(lg.clone())
        toks.append(qwen_text.greedy(lg))
        # the exchange of per-rank maxima picks the same id as a greedy pass over the gathered logits
        assert tp_oracle.greedy_by_exchange(lg[rank * n_l:(rank + 1) * n_l], rank, world) == toks[-1]
        if s + 1 < steps:
            lg = o.forward([toks[-1]])
    # ties across ranks and inside a rank: the lowest global id wins
    tie = torch.zeros(cfg.vocab)
    tie[[n_l - 1, n_l + 3, n_l + 5, cfg.vocab - 1]] = 7.0
    assert tp_oracle.greedy_by_exchange(tie[rank * n_l:(rank + 1) * n_l], rank, world) == n_l - 1 == qwen_text.greedy(tie)
    torch.save({"tokens": toks, "logits": torch.stack(logits)}, os.path.join(out_dir, f"rank{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


def gpu_rank(rank, world, port, cfg_kw, seed, n_prompt, steps, out_dir, use_graph, fused=False):
    """One GPU per rank: the CUDA backend with tp_size = world, NCCL between the ranks."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import cabi
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)      # host plumbing for the 128-byte id
    cfg = synth.tiny_config(**cfg_kw)
    w = synth.make_weights(cfg, seed=seed)
    prompt = synth.make_token_ids(n_prompt, seed=seed, vocab=cfg.vocab)
    box = [cabi.tp_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(box, src=0)
    be = cabi.Backend(cfg, device_id=rank, tp_rank=rank, tp_size=world)
    be.tp_init(box[0])
    be.load_weights(w)
    be.alloc_slot(0, 256)
    be.set_sampling(0.0, 1.0, 0)
    if fused:        # decode all-reduces inside the GEMVs over peer memory: exchange the IPC handles, then a barrier
        handles = [None] * world
        dist.all_gather_object(handles, be.tp_peer_export())
        be.tp_peer_import(handles)
        dist.barrier()
    pos3 = None
    if cfg.mrope_section is not None:
        pos3 = [list(range(n_prompt))] * 3
    toks, logits = cabi.generate(be, 0, prompt, steps, pos3=pos3, use_graph=use_graph, collect_logits=True)
    free, _ = cabi.generate(be, 0, prompt, steps, pos3=pos3, use_graph=use_graph)
    torch.save({"tokens": toks, "free": free, "logits": torch.from_numpy(__import__("numpy").stack(logits))}, os.path.join(out_dir, f"rank{rank}.pt"))
    dist.barrier()
    be.close()
    dist.destroy_process_group()


def gpu_vit_rank(rank, world, port, vit_kw, grids, seed, out_dir):
    """Vision encoder with its windows sharded over the tensor-parallel ranks (every rank returns the whole output)."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import cabi
    from oracle import qwen_vit
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    cfg = synth.tiny_config(num_layers=1, hidden=256, q_heads=4, kv_heads=2, intermediate=256, vocab=1000)
    box = [cabi.tp_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(box, src=0)
    be = cabi.Backend(cfg, device_id=rank, tp_rank=rank, tp_size=world)
    be.tp_init(box[0])
    vcfg = qwen_vit.VitConfig(**vit_kw)
    w = qwen_vit.make_weights(vcfg, seed=seed)
    px = qwen_vit.make_pixels(vcfg, grids, seed=seed)
    enc = cabi.VitEncoder(be, vcfg, max_patches=px.shape[0])
    enc.load_weights(w)
    out = torch.zeros(px.shape[0] // 4, vcfg.out_hidden, dtype=torch.bfloat16, device="cuda")
    for _ in range(2):                      # twice: buffers and collectives are reusable
        enc.encode(px.cuda(), grids, out)
        be.synchronize()
    torch.save(out.float().cpu(), os.path.join(out_dir, f"vit_rank{rank}.pt"))
    dist.barrier()
    enc.close()
    be.close()
    dist.destroy_process_group()


def gpu_engine_rank(rank, world, engine_json, prompt, out_dir):
    """Public API on several GPUs: every rank builds edge_fm.EdgeFM from the same JSON (runtime.tensor_parallel = world)
    and issues the same request; the ranks meet through the rendezvous directory named in the JSON."""
    os.environ.update(EFM_TP_RANK=str(rank), LOCAL_RANK=str(rank), NCCL_NVLS_ENABLE="0")
    import cabi
    if cabi.PY_DIR not in sys.path:
        sys.path.insert(0, cabi.PY_DIR)
    import edge_fm
    eng = edge_fm.EdgeFM(engine_json)
    outs = []
    for _ in range(2):
        req = edge_fm.Request(0, prompt)
        req.set_ignore_stop_tokens(True)
        outs.append(list(eng.generate(req).token_ids()))
    torch.save({"tokens": outs[0], "again": outs[1], "metrics": dict(eng.last_generate_metrics())}, os.path.join(out_dir, f"engine_rank{rank}.pt"))
    del eng
