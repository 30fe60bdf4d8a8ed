"""Benchmark of the single-request generate() hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--config 0..4]

Without --config the workload is configuration 3, the one the benchmark partitions: a Qwen2.5-VL-7B-shaped
random bf16 model, one 1288x728 image (4784 patches -> 1196 tokens through the vision encoder) + 128 text
tokens, INT8 prefill attention, 256 generated tokens at batch 1.  One "step" is one request: encode + prefill +
sample + 255 decode steps.  N = 1 runs it on one GPU; N > 1 (one process per GPU under torch.distributed.run)
runs the SAME request tensor parallel over the N ranks (heads + MLP columns + vocabulary rows; strong scaling).
  value  decode tok/s from CUDA events on the context stream around the decode phase (inputs resident);
  e2e    tokens/s of edge_fm.EdgeFM.generate() with host pixels / ids in and host ids out;
  per_config (N = 1 only)  a short pass over configurations 0, 1, 2 and 4 on the same GPU, plus configurations 1 and 3
             with the decode pass on group-wise INT4 weights ("1_int4", "3_int4").
--config k runs configuration k alone (0-2 and 4: replicas when N > 1).  Prints exactly one JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import datetime
import json
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for p in (ROOT, os.path.join(ROOT, "tests"), os.path.join(ROOT, "edge-fm-x_b200", "python")):
    if p not in sys.path:
        sys.path.insert(0, p)

METRIC, UNIT = "decode_tokens_per_second_batch1", "tok/s"
# DRAM bytes (read + write) of the four per-layer GEMV launches of one decode step: constants taken from one ncu
# capture per configuration (summaries under profiles/), not re-measured by this script.
NCU_LAYER_GEMV_DRAM_BYTES = {1: 6.33984e6 + 4.758528e6 + 55.090432e6 + 77.824e3 + 27.579904e6,
                             3: 33.099264e6 + 25.752576e6 + 271.638784e6 + 168.704e3 + 135.918848e6 + 327.168e3}
NAMES = {0: "qwen2.5-0.5b", 1: "qwen2.5-1.5b", 2: "qwen2.5-vl-3b-llm", 3: "qwen2.5-vl-7b-llm"}
HEADLINE = 3


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        return float(json.load(open(path))["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi clock / throttle samples of one GPU while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu):
        self.gpu, self.rows, self.proc = gpu, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.gpu), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", "200"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=3)
            except Exception:
                self.proc.kill()
        sm = sorted(float(r[1]) for r in self.rows if len(r) >= 9 and r[1].replace(".", "").isdigit())
        mx = [float(r[2]) for r in self.rows if len(r) >= 9 and r[2].replace(".", "").isdigit()]
        reasons = set()
        for r in self.rows:
            if len(r) >= 9:
                for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(name)
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def workload(cfg_id):
    from oracle import synth
    cfg = synth.CONFIGS[cfg_id]
    prefix_n, prompt_n, steps, temp, top_p = synth.WORKLOADS[cfg_id]
    ids = synth.make_token_ids(prefix_n + prompt_n, seed=0)
    return cfg, ids[:prefix_n], ids, steps, temp, top_p


def vlm_request(cfg_id, cfg):
    from oracle import synth
    return synth.vlm_request(cfg_id)


def workload_text(cfg_id, gen_tokens=None):
    """The workload sentence of configurations 0-3, the same in both arms (the reference arm samples its decode steps)."""
    cfg, prefix, ids, gen, temp, top_p = workload(cfg_id)
    gen = gen_tokens or gen
    if cfg.mrope_section is None:
        return (f"{NAMES[cfg_id]}: {len(prefix)}-token resident prefix + {len(ids) - len(prefix)}-token prompt, "
                f"{gen} generated tokens, batch 1, temperature {temp}, top_p {top_p}")
    vlm = vlm_request(cfg_id, cfg)
    n_patches = sum(t * h * w for t, h, w in vlm["grids"])
    n_text = len(vlm["ids"]) - vlm["n_img"]
    if cfg_id == 3:
        return (f"{NAMES[cfg_id]}: 1288x728 image ({n_patches} patches -> {vlm['n_img']} tokens through the vision encoder) + {n_text} text "
                f"tokens = {len(vlm['ids'])}-token prompt, {gen} generated tokens, batch 1, temperature {temp}, top_p {top_p}")
    return (f"{NAMES[cfg_id]}: 448x448 image ({n_patches} patches -> {vlm['n_img']} tokens through the vision encoder) + {n_text} text "
            f"tokens, {gen} generated tokens, batch 1, temperature {temp}, top_p {top_p}")


def vit_flops(vcfg, grids):
    """Algorithmic flops of one encode: 2 m n k per GEMM, 4 D per (query, visible key, head)."""
    from oracle import qwen_vit
    plan = qwen_vit.make_plan(vcfg, grids)
    n = plan.cu_full[-1]
    H, I, M = vcfg.hidden, vcfg.intermediate, vcfg.hidden * vcfg.merge ** 2
    win = sum((b - a) ** 2 for a, b in zip(plan.cu_window[:-1], plan.cu_window[1:]))
    full = sum((b - a) ** 2 for a, b in zip(plan.cu_full[:-1], plan.cu_full[1:]))
    per_layer = 2 * n * (3 * H * H + H * H + 3 * H * I)
    att = 4 * H * (win * (vcfg.depth - len(vcfg.fullatt)) + full * len(vcfg.fullatt))
    return 2 * n * vcfg.patch_dim * H + vcfg.depth * per_layer + att + 2 * (n // vcfg.merge ** 2) * (M * M + M * vcfg.out_hidden)


def prefill_flops(cfg, s, prefix):
    H, I = cfg.hidden, cfg.intermediate
    qd, kvd = cfg.q_heads * cfg.head_dim, cfg.kv_heads * cfg.head_dim
    lin = 2 * s * (H * (qd + 2 * kvd) + qd * H + 3 * H * I)
    att = 4 * qd * sum(prefix + i + 1 for i in range(s))
    return cfg.num_layers * (lin + att) + 2 * cfg.vocab * H


def tensor_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        return float(json.load(open(path))["bf16_tflops"]), "measured"
    return 1590.0, "fallback"


def tensor_report(flops, ms):
    peak, kind = tensor_peak()
    tf = flops / (ms * 1e-3) / 1e12
    return {"ms": ms, "tflop": flops / 1e12, "tflops": tf, "frac_of_bf16_peak": tf / peak, "peak": peak, "peak_kind": kind}


def scratch_dir(rank, need_gb):
    """A fresh directory for a synthetic checkpoint: memory-backed when it has the room, else the default temp dir."""
    base = None
    try:
        st = os.statvfs("/dev/shm")
        if st.f_bavail * st.f_frsize > (need_gb + 4) * 2 ** 30:
            base = "/dev/shm"
    except OSError:
        pass
    return tempfile.mkdtemp(prefix=f"efm_bench_{rank}_", dir=base)


# --------------------------------------------------------------------------------------------------
# CPU arm: the reference has no CPU implementation of this path (it throws without CUDA) and cannot be built here,
# so both `--impl reference` and the cpu_baseline object time the fp32 torch-CPU restatement on the host cores.
class CpuDecode:
    """The restatement positioned at the workload's REAL context: the prompt is prefilled once (outside any timed
    region; image rows are seeded noise of the embeddings' scale, since decode time does not depend on their
    values), then decode steps are timed and the cache rolled back."""

    def __init__(self, cfg_id, weights=None):
        import torch
        from oracle import qwen_text, synth
        self.torch = torch
        self.cfg = cfg = synth.CONFIGS[cfg_id]
        self.cores = os.cpu_count() or 1
        torch.set_num_threads(self.cores)
        w = weights if weights is not None else synth.make_weights(cfg, seed=0)
        self.o = qwen_text.QwenTextOracle(cfg, w, "exact_fp32")
        del w
        if cfg.mrope_section is not None:
            vlm = vlm_request(cfg_id, cfg)
            ids, pos = vlm["ids"], torch.tensor(vlm["pos"])
            g = torch.Generator().manual_seed(0)
            embeds = torch.randn(vlm["n_img"], cfg.hidden, generator=g) * 0.02
            self.first_pos = vlm["last"] + 1
        else:
            _, _, ids, _, _, _ = workload(cfg_id)
            pos, embeds, self.first_pos = None, None, None
        self.ctx = len(ids)
        self.tok = ids[-1]
        t0 = time.perf_counter()
        with torch.no_grad():
            self.o.forward(ids, embeds=embeds, embed_token_id=cfg.vocab if embeds is not None else -1, position_ids=pos)
        self.prefill_s = time.perf_counter() - t0

    def decode(self, n):
        torch, o = self.torch, self.o
        n0 = o.kv_len
        with torch.no_grad():
            for i in range(n):
                p3 = None if self.first_pos is None else torch.full((3, 1), self.first_pos + i)
                o.forward([self.tok], position_ids=p3)
        o.truncate(n0)


def run_reference(args, rank):
    """One bench step = a bounded sample: `sample_tokens` decode steps at the workload's full context."""
    if rank != 0:
        return
    cpu = CpuDecode(args.config)
    sample_tokens = 1 if args.config == 3 else 2
    for _ in range(args.warmup):
        cpu.decode(sample_tokens)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu.decode(sample_tokens)
    dt = time.perf_counter() - t0
    value = args.steps * sample_tokens / dt
    sample = (f"{sample_tokens} decode step(s) per bench step at context {cpu.ctx} (the workload's own), fp32 torch-CPU restatement; "
              f"prompt prefilled once outside the timed region ({cpu.prefill_s:.1f} s)")
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True,
            "scaling": "strong" if args.config == 3 else "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": workload_text(args.config),
                       "parallelism": f"{cpu.cores} host threads",
                       "reference_path": f"CPU restatement of the reference path, decode steps at context {cpu.ctx} (the reference "
                                         "itself has no CPU implementation of token generation and cannot be built here)"},
            "cpu_baseline": {"value": value, "unit": UNIT, "cores": cpu.cores, "kind": "port", "sample": sample,
                             "prefill_s": cpu.prefill_s},
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def cpu_baseline(cfg_id, weights=None, budget_s=20.0):
    cpu = CpuDecode(cfg_id, weights)
    cpu.decode(1)
    n, t0 = 0, time.perf_counter()
    while n < 64 and (n < 8 or time.perf_counter() - t0 < budget_s):
        cpu.decode(1)
        n += 1
    dt = time.perf_counter() - t0
    return {"value": n / dt, "unit": UNIT, "cores": cpu.cores, "kind": "port", "prefill_s": cpu.prefill_s,
            "sample": f"{n} decode steps at context {cpu.ctx} (the workload's own), fp32 torch-CPU restatement, all host threads"}


# --------------------------------------------------------------------------------------------------
class _Solo:
    """torch.distributed stand-in for a single process."""
    class ReduceOp:
        MAX = None

    @staticmethod
    def barrier():
        pass

    @staticmethod
    def all_reduce(t, op=None):
        pass

    @staticmethod
    def broadcast_object_list(box, src=0):
        pass

    @staticmethod
    def all_gather_object(out, obj):
        out[0] = obj

    @staticmethod
    def destroy_process_group():
        pass


def draw_weights_on_device(cfg, be, keep_host, int4=False):
    """Seeded weights drawn tensor by tensor on the GPU (identical on every rank: same generator, same order), handed
    to the backend from device memory; rank 0 may keep host copies for the checkpoint the public-API engine loads.
    int4: every linear is also quantised (group-wise, on the device) and handed over as the decode-pass checkpoint."""
    import torch
    from oracle import synth
    if int4:
        from oracle import int4 as int4_tools
        linear = tuple("." + n + ".weight" for n in int4_tools.LINEARS)
    g = torch.Generator(device="cuda")
    g.manual_seed(0)
    host = {}
    for name, shape, kind in synth.weight_names(cfg):       # one tensor at a time: the whole model never sits twice in HBM
        t = torch.randn(shape, generator=g, device="cuda", dtype=torch.float32) * 0.02
        if kind == "n":
            t += 1.0
        t = t.to(torch.bfloat16)
        be.load_weights_partial({name: t})
        if int4 and (name.endswith(linear) or name == "lm_head.weight" or (cfg.tied and name == "model.embed_tokens.weight")):
            q, sc = int4_tools.quantize(t)
            stem = "lm_head" if name in ("lm_head.weight", "model.embed_tokens.weight") else name[:-len(".weight")]
            be.load_decode_weights_int4({stem + ".qweight": int4_tools.pack(q), stem + ".scaling_factors": sc})
            del q, sc
        if keep_host:
            host[name] = t.cpu()
        del t
    be.finalize()
    return host


def run_tp(args, rank, world, local_rank):
    """Config 3 (7B-class): ONE request, tensor parallel over all ranks (strong scaling); one rank = the plain
    single-GPU path."""
    import torch
    import torch.distributed as dist
    import cabi
    from oracle import qwen_vit, synth
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(local_rank)
    if world > 1:
        # a short collective timeout: a rank that raises must end the job, not leave the others waiting for ten minutes
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank), timeout=datetime.timedelta(seconds=240))
    else:
        dist = _Solo
    cfg, prefix, ids, gen_tokens, temp, top_p = workload(args.config)
    if args.tokens:
        gen_tokens = args.tokens
    vlm = vlm_request(args.config, cfg)
    ids, pos = vlm["ids"], vlm["pos"]
    max_tokens = len(ids) + gen_tokens + 8
    int4 = bool(args.int4)
    if int4 and world > 1:
        raise SystemExit("--int4 runs on one GPU (the tensor-parallel decode step streams bf16 weights)")
    want_e2e = not args.no_e2e and not int4
    want_cpu = world == 1 and not args.no_cpu and not int4
    t_setup = time.perf_counter()
    be = cabi.Backend(cfg, max_prefill_tokens=min(2048, max_tokens), max_response_tokens=gen_tokens + 8,
                      device_id=local_rank, tp_rank=rank, tp_size=world)
    if world > 1:
        box = [cabi.tp_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(box, src=0)
        be.tp_init(box[0])
    host_w = draw_weights_on_device(cfg, be, keep_host=rank == 0 and (want_e2e or want_cpu), int4=int4)
    be.alloc_slot(0, max_tokens)
    fused = world > 1 and args.tp_exchange == "peer"
    if fused:        # the decode step's all-reduces inside the GEMVs, over peer memory (CUDA IPC handles via the host)
        handles = [None] * world
        dist.all_gather_object(handles, be.tp_peer_export())
        be.tp_peer_import(handles)
        dist.barrier()
    if args.prefill_attention == "int8":        # the benchmark's configuration 3 prefills with the INT8 attention scheme
        be.set_prefill_attention(1)
    be.set_sampling(temp, top_p, 0)
    be.set_prefill_graph(True)       # as the engine does with runtime.use_cuda_graph: the request's prefill shape is captured once
    be.capture_decode(0)
    # vision encoder on the text context's stream; its windows are sharded over the ranks
    n_patches = sum(t * h * w for t, h, w in vlm["grids"])
    enc = cabi.VitEncoder(be, vlm["vcfg"], max_patches=n_patches)
    enc.load_weights(qwen_vit.make_weights(vlm["vcfg"], seed=0, device="cuda"))
    pixels = qwen_vit.make_pixels(vlm["vcfg"], vlm["grids"], seed=0)
    pixels_host = pixels.pin_memory()
    pixels_dev = pixels.cuda()
    embeds = torch.zeros(vlm["n_img"], cfg.hidden, dtype=torch.bfloat16, device="cuda")
    be.synchronize()

    setup_s = time.perf_counter() - t_setup
    mp = [vlm["last"] + 1] * 3

    def one_request():
        be.event_record(0)
        enc.encode(pixels_dev, vlm["grids"], embeds)
        be.event_record(3)
        be.prefill(0, ids, kv_offset=0, embeds=embeds, embed_token_id=vlm["embed_id"], pos3=pos, sample=True)
        be.event_record(1)
        be.decode_begin(0, len(ids), mp, 1)
        be.decode_steps(gen_tokens - 1, True)
        be.event_record(2)
        toks = be.read_tokens(0, gen_tokens)              # host ids out (one D2H + sync)
        return be.elapsed_ms(3, 1), be.elapsed_ms(1, 2), toks, be.elapsed_ms(0, 3)

    pt = torch.tensor(pos, dtype=torch.int32)

    def e2e_request(engine, enc2, eb):       # host pixels -> vision encoder (C ABI) -> embeddings stay on the device -> public generate()
        import edge_fm
        enc2.encode(pixels_host, vlm["grids"], embeds)
        eb.synchronize()
        req = edge_fm.Request(0, ids, edge_fm.Tensor(embeds.data_ptr(), [vlm["n_img"], cfg.hidden], edge_fm.DType.BFloat16,
                                                     edge_fm.Device.GPU, local_rank),
                              vlm["embed_id"], edge_fm.Tensor(pt.data_ptr(), [3, len(ids)], edge_fm.DType.Int32, edge_fm.Device.CPU),
                              [vlm["last"]] * 3, device=edge_fm.Device.GPU, device_id=local_rank)
        req.set_ignore_stop_tokens(True)
        return list(engine.generate(req).token_ids())

    for _ in range(args.warmup):
        one_request()
    sampler = ClockSampler(local_rank)
    sampler.start()
    launches0 = be.launch_count()
    dist.barrier()
    torch.cuda.synchronize()
    pre_ms = dec_ms = vit_ms = 0.0
    for _ in range(args.steps):
        a, b, tokens, v = one_request()
        pre_ms += a
        dec_ms += b
        vit_ms += v
    dist.barrier()
    torch.cuda.synchronize()
    launches = be.launch_count() - launches0
    clocks = sampler.stop()
    torch.cuda.set_device(local_rank)
    local = torch.tensor([dec_ms, pre_ms, vit_ms], dtype=torch.float64, device=torch.device("cuda", local_rank))
    dist.all_reduce(local, op=dist.ReduceOp.MAX)
    dec_ms, pre_ms, vit_ms = [float(x) for x in local.tolist()]
    dec_steps = args.steps * (gen_tokens - 1)
    step_ms = dec_ms / dec_steps
    step_bytes = be.decode_step_bytes(len(ids) + gen_tokens // 2)          # this rank's share
    breakdown = None
    if world == 1 or fused:      # per-kernel device time of a few un-overlapped steps (every rank takes part)
        be.decode_begin(0, len(ids), mp, 1)
        bd = be.decode_breakdown(4)
        Lc = cfg.num_layers
        breakdown = {k: round(v / (4 * (Lc if k not in ("lm_head", "sampler") else 1)) * 1e3, 2) for k, v in bd.items()}
    peak, peak_kind = peaks()
    achieved = step_bytes / (step_ms * 1e-3) / 1e9
    traffic = None
    if world == 1 and not int4 and args.config in NCU_LAYER_GEMV_DRAM_BYTES:      # measured for the layer GEMVs, algorithmic for the rest
        qD, kvD, H, I = cfg.q_heads * cfg.head_dim, cfg.kv_heads * cfg.head_dim, cfg.hidden, cfg.intermediate
        layer_alg = 2 * ((qD + 2 * kvD) * H + qD * H + 3 * I * H)
        traffic = step_bytes + cfg.num_layers * (NCU_LAYER_GEMV_DRAM_BYTES[args.config] - layer_alg)
    line = None
    if rank == 0:
        line = {"metric": METRIC, "value": dec_steps / (dec_ms / 1e3), "unit": UNIT, "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": (vit_ms + pre_ms + dec_ms) / args.steps, "higher_is_better": True,
                "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                "config": {"workload": workload_text(args.config, gen_tokens),
                           "parallelism": "single GPU" if world == 1 else f"tp{world} (heads + MLP columns + vocab rows; decode all-reduce: " +
                                          ("fused into the GEMVs over peer memory" if fused else "NCCL in the decode graph") +
                                          "; prefill: reduce-scatter + all-gather over peer stores; vision windows sharded)",
                           "prefill_attention": args.prefill_attention,
                           "l2_policy": "weights streamed per decode step exceed L2 (%.2f GB per GPU vs 126 MB)" % (step_bytes / 1e9),
                           "cuda_graph": True},
                "decode_ms_per_token": step_ms, "prefill_ms": pre_ms / args.steps, "vit_ms": vit_ms / args.steps,
                "ttft_ms": (pre_ms + vit_ms) / args.steps,
                "prefill": tensor_report(prefill_flops(cfg, len(ids), 0) / world, pre_ms / args.steps),
                "vit": tensor_report(vit_flops(vlm["vcfg"], vlm["grids"]) / world, vit_ms / args.steps),
                "setup_s": setup_s,
                "gpu_launches": launches, "clocks": clocks,
                "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                             "traffic": traffic,
                             "traffic_source": "constants from one ncu capture (dram__bytes_read+write of the per-layer GEMV launches, "
                                               "summary under profiles/) + algorithmic bytes of lm_head, attention and vectors" if traffic else None,
                             "peak_kind": peak_kind,
                             "weights": "int4 group-128 (decode pass), bf16 (prefill)" if int4 else "bf16",
                             "launch": "one decode step on one rank (CUDA graph: 5 kernels per layer + lm_head + sampler; the ranks exchange inside the kernels)",
                             "bytes_per_launch": step_bytes, "us_per_launch": step_ms * 1e3,
                             "frac_of_nominal_8tbs": achieved / 8000.0},
                "tokens_head": tokens[:8]}
        if breakdown is not None:
            line["roofline"]["kernel_us_unoverlapped"] = breakdown
    enc.close()
    be.close()
    del be, enc
    torch.cuda.empty_cache()
    dist.barrier()

    # ---- end to end through the public API: every rank builds edge_fm.EdgeFM from the same JSON; the vision encoder is
    #      created on the ENGINE's device backend (EdgeFM.backend_handle), so one context, one stream and one
    #      tensor-parallel communicator serve the whole request
    if want_e2e:
        import edge_fm
        box = [scratch_dir(rank, 16) if rank == 0 else None]
        dist.broadcast_object_list(box, src=0)
        tmp = box[0]
        model_dir = os.path.join(tmp, "model")
        if rank == 0:
            synth.write_checkpoint(model_dir, cfg, host_w)
            eng_path = synth.write_engine_config(os.path.join(tmp, "engine.json"), model_dir, model_name="Qwen2.5-VL", prefix_ids=[],
                                                 max_tokens=max_tokens, max_new_tokens=gen_tokens, temperature=temp, top_p=top_p,
                                                 seed=0, use_cuda_graph=True, device_id=local_rank)
            ej = json.load(open(eng_path))
            ej["runtime"]["prefill_attention"] = args.prefill_attention
            if world > 1:
                ej["runtime"]["tensor_parallel"] = world
                ej["runtime"]["tp_rendezvous"] = os.path.join(tmp, "meet")
            json.dump(ej, open(eng_path, "w"))
        dist.barrier()
        os.environ["EFM_TP_RANK"] = str(rank)
        os.environ["LOCAL_RANK"] = str(local_rank)
        engine = edge_fm.EdgeFM(os.path.join(tmp, "engine.json"))
        dist.barrier()
        if rank == 0:
            shutil.rmtree(tmp, ignore_errors=True)
        eb = EngineBackend(engine)
        enc2 = cabi.VitEncoder(eb, vlm["vcfg"], max_patches=n_patches)
        enc2.load_weights(qwen_vit.make_weights(vlm["vcfg"], seed=0, device="cuda"))
        eb.synchronize()
        e2e_tokens = None
        for _ in range(max(2, min(3, args.warmup))):          # first request eager, second captures the prefill graph
            e2e_tokens = e2e_request(engine, enc2, eb)
        dist.barrier()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            e2e_tokens = e2e_request(engine, enc2, eb)
        dist.barrier()
        torch.cuda.synchronize()
        wall = torch.tensor([time.perf_counter() - t0], dtype=torch.float64, device=torch.device("cuda", local_rank))
        dist.all_reduce(wall, op=dist.ReduceOp.MAX)
        wall_max = float(wall.item())
        m = engine.last_generate_metrics()
        if rank == 0:
            line["wall_s"] = wall_max
            line["e2e"] = {"value": args.steps * gen_tokens / wall_max, "unit": UNIT,
                           "h2d_bytes_per_step": 16 * len(ids) + pixels.numel() * 2, "d2h_bytes_per_step": 4 * gen_tokens + 32,
                           "api": "efm_b200_vit_encode on the engine's backend (host pixels) -> edge_fm.EdgeFM.generate (host ids in / out)" +
                                  ("" if world == 1 else f", runtime.tensor_parallel = {world}"),
                           "engine_decode_tok_s": m.get("decode_tokens_per_second"), "engine_prefill_ms": m.get("prefill_ms"),
                           "engine_metrics": {k: round(float(v), 3) for k, v in m.items()}}
            line["e2e_tokens_equal"] = e2e_tokens == tokens
        enc2.close()
        engine = None
        dist.barrier()
    if world > 1:
        dist.destroy_process_group()
    if rank == 0 and want_cpu:
        torch.cuda.empty_cache()
        line["cpu_baseline"] = cpu_baseline(args.config, host_w)
    return line


class EngineBackend:
    """The device backend of an edge_fm.EdgeFM engine seen through the C ABI (for the vision encoder that feeds it)."""

    def __init__(self, engine):
        import cabi
        self.L = cabi.lib()
        self.ctx = cabi.P(engine.backend_handle())
        if not self.ctx:
            raise RuntimeError("the engine has no device backend handle")

    def check(self, st, what=""):
        if st != 0:
            raise RuntimeError(f"{what} failed ({st}): {self.L.efm_b200_last_error(self.ctx).decode()}")

    def synchronize(self):
        self.check(self.L.efm_b200_synchronize(self.ctx), "synchronize")


def run_text(args, cfg_id, rank, world, local_rank, *, steps, warmup, want_cpu, dist=None, int4=False):
    """Configurations 0-2 on one GPU (world > 1: independent replicas, one per rank).  int4: the decode pass runs on a
    group-wise INT4 copy of every linear (two checkpoints: bf16 for prefill, INT4 for decode); C ABI only."""
    import torch
    import cabi
    from oracle import synth
    torch.cuda.set_device(local_rank)
    cfg, prefix, ids, gen_tokens, temp, top_p = workload(cfg_id)
    if args.tokens:
        gen_tokens = args.tokens
    vlm = vlm_request(cfg_id, cfg) if cfg.mrope_section is not None else None
    if vlm is not None:
        ids = vlm["ids"]
    prompt_n = len(ids) - len(prefix)
    max_tokens = len(ids) + gen_tokens + 8
    pos = vlm["pos"] if vlm is not None else None

    t_setup = time.perf_counter()
    w = synth.make_weights(cfg, seed=0, device="cuda")
    be = cabi.Backend(cfg, max_prefill_tokens=min(2048, max_tokens), max_response_tokens=gen_tokens + 8, device_id=local_rank)
    if int4:
        from oracle import int4 as int4_tools
        packed, _ = int4_tools.quantize_checkpoint(w, cfg.num_layers, lm_head=True)     # quantised on the device
        be.load_weights_partial(w)
        be.load_decode_weights_int4(packed)
        be.finalize()
        del packed
    else:
        be.load_weights(w)
    be.alloc_slot(0, max_tokens)
    be.set_sampling(temp, top_p, 0)
    if prefix:
        be.prefill(0, prefix, kv_offset=0, pos3=None if pos is None else [r[:len(prefix)] for r in pos], sample=False)
    be.set_prefill_graph(True)       # as the engine does with runtime.use_cuda_graph: the request's prefill shape is captured once
    be.capture_decode(0)
    enc = None
    if vlm is not None:
        from oracle import qwen_vit
        n_patches = sum(t * h * w_ for t, h, w_ in vlm["grids"])
        enc = cabi.VitEncoder(be, vlm["vcfg"], max_patches=n_patches)
        enc.load_weights(qwen_vit.make_weights(vlm["vcfg"], seed=0, device="cuda"))
        pixels = qwen_vit.make_pixels(vlm["vcfg"], vlm["grids"], seed=0)
        pixels_host, pixels_dev = pixels.pin_memory(), pixels.cuda()
        embeds = torch.zeros(vlm["n_img"], cfg.hidden, dtype=torch.bfloat16, device="cuda")
    be.synchronize()

    # public API engine for the end-to-end leg (weights travel through a safetensors checkpoint)
    engine, tmp = None, None
    if not args.no_e2e and not int4:
        import edge_fm
        tmp = scratch_dir(rank, 8)
        model_dir = synth.write_checkpoint(os.path.join(tmp, "model"), cfg, w)
        name = "Qwen2.5-VL" if cfg.mrope_section is not None else "Qwen2.5"
        eng_cfg = synth.write_engine_config(os.path.join(tmp, "engine.json"), model_dir, model_name=name, prefix_ids=prefix,
                                            max_tokens=max_tokens, max_new_tokens=gen_tokens, temperature=temp, top_p=top_p,
                                            seed=0, use_cuda_graph=True, device_id=local_rank)
        engine = edge_fm.EdgeFM(eng_cfg)
        shutil.rmtree(tmp, ignore_errors=True)
    host_w = {k: v.cpu() for k, v in w.items()} if want_cpu else None
    del w
    setup_s = time.perf_counter() - t_setup

    suffix = ids[len(prefix):]
    pos_suffix = None if pos is None else [r[len(prefix):] for r in pos]
    mp = None if vlm is None else [vlm["last"] + 1] * 3

    def one_request():
        be.event_record(0)
        if enc is not None:
            enc.encode(pixels_dev, vlm["grids"], embeds)
        be.event_record(3)
        if enc is not None:
            be.prefill(0, suffix, kv_offset=len(prefix), embeds=embeds, embed_token_id=vlm["embed_id"], pos3=pos_suffix, sample=True)
        else:
            be.prefill(0, suffix, kv_offset=len(prefix), pos3=pos_suffix, sample=True)
        be.event_record(1)
        be.decode_begin(0, len(ids), mp, 1)
        be.decode_steps(gen_tokens - 1, True)
        be.event_record(2)
        be.synchronize()
        return be.elapsed_ms(3, 1), be.elapsed_ms(1, 2), be.elapsed_ms(0, 3)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(warmup):
        one_request()
    sampler = ClockSampler(local_rank)
    sampler.start()
    launches0 = be.launch_count()
    barrier()
    t0 = time.perf_counter()
    pre_ms, dec_ms, vit_ms = 0.0, 0.0, 0.0
    for _ in range(steps):
        a, b, v = one_request()
        pre_ms += a
        dec_ms += b
        vit_ms += v
    barrier()
    wall_s = time.perf_counter() - t0
    launches = be.launch_count() - launches0
    tokens = be.read_tokens(0, gen_tokens)

    # end to end through the public API: host ids in, host ids out
    def e2e_request():
        if vlm is None:
            req = edge_fm.Request(0, ids)
        else:       # host pixels -> vision encoder (C ABI) -> embeddings stay on the device -> public generate()
            enc.encode(pixels_host, vlm["grids"], embeds)
            be.synchronize()
            pt = torch.tensor(pos, dtype=torch.int32)
            req = edge_fm.Request(0, ids, edge_fm.Tensor(embeds.data_ptr(), [vlm["n_img"], cfg.hidden], edge_fm.DType.BFloat16,
                                                         edge_fm.Device.GPU, local_rank),
                                  vlm["embed_id"],
                                  edge_fm.Tensor(pt.data_ptr(), [3, len(ids)], edge_fm.DType.Int32, edge_fm.Device.CPU), [vlm["last"]] * 3,
                                  device=edge_fm.Device.GPU, device_id=local_rank)
        req.set_ignore_stop_tokens(True)
        return list(engine.generate(req).token_ids())
    e2e_s, e2e_tokens, m = None, None, {}
    if engine is not None:
        for _ in range(max(2, min(3, warmup))):        # first request eager, second captures the prefill graph
            e2e_tokens = e2e_request()
        barrier()
        t1 = time.perf_counter()
        for _ in range(steps):
            e2e_tokens = e2e_request()
        barrier()
        e2e_s = time.perf_counter() - t1
        m = engine.last_generate_metrics()
    clocks = sampler.stop()

    # per-kernel device time of a few un-overlapped steps (after the timed region)
    be.decode_begin(0, len(ids), mp, 1)
    breakdown = be.decode_breakdown(4)
    step_bytes = be.decode_step_bytes(len(ids) + gen_tokens // 2)

    dec_steps = steps * (gen_tokens - 1)
    torch.cuda.set_device(local_rank)
    local = torch.tensor([dec_ms, pre_ms, wall_s, e2e_s or 0.0, vit_ms], dtype=torch.float64, device=torch.device("cuda", local_rank))
    if dist is not None:
        dist.all_reduce(local, op=dist.ReduceOp.MAX)
    dec_ms_max, pre_ms_max, wall_max, e2e_max, vit_ms_max = [float(x) for x in local.tolist()]
    value = world * dec_steps / (dec_ms_max / 1e3)
    step_ms = dec_ms_max / dec_steps
    peak, peak_kind = peaks()
    achieved = step_bytes / (step_ms * 1e-3) / 1e9
    H, I, L = cfg.hidden, cfg.intermediate, cfg.num_layers
    qd, kvd = cfg.q_heads * cfg.head_dim, cfg.kv_heads * cfg.head_dim
    kbytes = {"qkv": (qd + 2 * kvd) * H * 2, "o_proj": H * qd * 2, "gate_up": 2 * I * H * 2, "down_proj": H * I * 2,
              "lm_head": cfg.vocab * H * 2}
    kernels = {}
    for k, ms in breakdown.items():
        n_launch = 4 * (L if k not in ("lm_head", "sampler") else 1)
        us = ms / n_launch * 1e3
        kernels[k] = {"us_per_launch": round(us, 2)}
        if k in kbytes:
            kernels[k]["gbs"] = round(kbytes[k] / (us * 1e-6) / 1e9, 1)
            kernels[k]["frac"] = round(kbytes[k] / (us * 1e-6) / 1e9 / peak, 3)
    traffic = None
    if int4:       # the bytes of the per-kernel table are those of the INT4 matrices
        w4 = lambda n: n // 2 + n // 128 * 2
        kbytes = {k: w4(v // 2) for k, v in kbytes.items()}
        for k, item in kernels.items():
            if k in kbytes:
                us = item["us_per_launch"]
                item["gbs"] = round(kbytes[k] / (us * 1e-6) / 1e9, 1)
                item["frac"] = round(kbytes[k] / (us * 1e-6) / 1e9 / peak, 3)
    if cfg_id in NCU_LAYER_GEMV_DRAM_BYTES and not int4:       # measured for the layer GEMVs, algorithmic for the rest of the step
        layer_alg = sum(v for k, v in kbytes.items() if k != "lm_head")
        traffic = step_bytes + L * (NCU_LAYER_GEMV_DRAM_BYTES[cfg_id] - layer_alg)
    line = None
    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": steps, "warmup": warmup,
            "ms_per_step": (vit_ms_max + pre_ms_max + dec_ms_max) / steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": workload_text(cfg_id, gen_tokens),
                       "parallelism": "single GPU" if world == 1 else f"{world} independent replicas",
                       "l2_policy": "weights streamed per decode step exceed L2 (%.2f GB vs 126 MB)" % (step_bytes / 1e9),
                       "cuda_graph": True},
            "decode_ms_per_token": step_ms, "prefill_ms": pre_ms_max / steps,
            "ttft_ms": (pre_ms_max + vit_ms_max) / steps, "wall_s": wall_max, "setup_s": setup_s,
            "prefill": tensor_report(prefill_flops(cfg, prompt_n, len(prefix)), pre_ms_max / steps),
            "gpu_launches": launches,
            "clocks": clocks,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": traffic,
                         "traffic_source": "constants from one ncu capture (dram__bytes_read+write of the per-layer GEMV launches, summary "
                                           "under profiles/) + algorithmic bytes of lm_head, attention and vectors" if traffic else None,
                         "peak_kind": peak_kind, "weights": "int4 group-128 (decode pass), bf16 (prefill)" if int4 else "bf16",
                         "launch": "one decode step (CUDA graph of %d kernel nodes: 5 per layer + lm_head + sampler)" % (5 * L + 2),
                         "bytes_per_launch": step_bytes, "us_per_launch": step_ms * 1e3, "frac_of_nominal_8tbs": achieved / 8000.0,
                         "kernels": kernels},
            "tokens_head": tokens[:8],
        }
        if e2e_s is not None:
            line["e2e"] = {"value": world * steps * gen_tokens / e2e_max, "unit": UNIT,
                           "h2d_bytes_per_step": 4 * prompt_n + (12 * len(ids) + pixels.numel() * 2 if vlm is not None else 0),
                           "d2h_bytes_per_step": 4 * gen_tokens + 32, "api": "edge_fm.EdgeFM.generate",
                           "engine_decode_tok_s": m.get("decode_tokens_per_second"), "engine_prefill_ms": m.get("prefill_ms"),
                           "engine_metrics": {k: round(float(v), 3) for k, v in m.items()}}
            line["e2e_tokens_equal"] = e2e_tokens == tokens
        if vlm is not None:
            line["vit_ms"] = vit_ms_max / steps
            line["vit"] = tensor_report(vit_flops(vlm["vcfg"], vlm["grids"]), vit_ms_max / steps)
    if enc is not None:
        enc.close()
    be.close()
    engine = None
    if rank == 0 and want_cpu:
        torch.cuda.empty_cache()
        line["cpu_baseline"] = cpu_baseline(cfg_id, host_w)
    return line


# --------------------------------------------------------------------------------------------------
# config 4: SmolVLA-shaped action chunk (chunks/s)
VLA_METRIC, VLA_UNIT = "action_chunks_per_second_batch1", "chunks/s"


def vla_flops(c):
    """Algorithmic flops of one chunk: 2*m*n*k per GEMM, 4*q*D*(visible keys) per query head per attention."""
    NV, Hv, P, n = c.n_images * c.patches, c.vit_hidden, c.prefix, c.chunk
    QD, KD, H, He = c.q_heads * c.head_dim, c.kv_heads * c.head_dim, c.hidden, c.expert_hidden
    vit = 2 * NV * Hv * c.patch_dim + c.vit_layers * (2 * NV * Hv * (4 * Hv + 2 * c.vit_mlp) + 4 * NV * c.patches * Hv)
    vit += 2 * c.n_images * c.image_tokens * H * Hv * c.shuffle ** 2
    vlm = c.layers * (2 * P * H * (QD + 2 * KD) + 2 * P * QD * H + 6 * P * H * c.mlp + 4 * P * P * QD)
    bridge = (c.layers // 2) * 2 * (2 * P * KD * KD)
    per_step = 2 * n * (c.action_dim * He + 2 * He * He + He * He + He * c.action_dim)
    for l in range(c.layers):
        per_step += 2 * n * He * (QD + (2 * KD if l % 2 == 0 else 0)) + 2 * n * QD * He + 6 * n * He * c.expert_mlp
        per_step += 4 * n * QD * (P + (n + 1) / 2 if l % 2 == 0 else P)
    return {"vision": vit, "prefix": vlm + bridge, "denoise": c.steps * per_step}


def vla_cpu_chunks_per_s(c, w, inp, steps):
    """The CPU restatement (oracle, exact_fp32, torch CPU threads) on full chunks of the same workload."""
    import torch
    from oracle import smolvla
    o = smolvla.VlaOracle(c, w, mode="exact_fp32")
    t0 = time.perf_counter()
    with torch.no_grad():
        for _ in range(steps):
            o.chunk(*inp)
    return steps / (time.perf_counter() - t0), torch.get_num_threads()


def vla_config_dict(c):
    return {"workload": f"smolvla-shaped chunk: {c.n_images} x {c.image_size}px images -> vision tower ({c.vit_layers} layers, "
                        f"hidden {c.vit_hidden}) -> {c.n_images * c.image_tokens} image tokens + {c.lang_tokens} prompt tokens + state = "
                        f"{c.prefix}-token prefix through a {c.layers}-layer backbone (hidden {c.hidden}); {c.steps} Euler steps of a "
                        f"{c.layers}-layer action expert (hidden {c.expert_hidden}) over {c.chunk} x {c.action_dim} actions; batch 1",
            "l2_policy": "weights read per chunk (about 0.7 GB) exceed L2 (126 MB)", "cuda_graph": True}


def run_vla_reference(args, rank):
    if rank != 0:
        return
    from oracle import smolvla
    c = smolvla.VlaConfig()
    w, inp = smolvla.make_weights(c, seed=0), smolvla.make_inputs(c, seed=0)
    vla_cpu_chunks_per_s(c, w, inp, max(1, args.warmup))
    t0 = time.perf_counter()
    v, cores = vla_cpu_chunks_per_s(c, w, inp, args.steps)
    ms = (time.perf_counter() - t0) / args.steps * 1e3
    sample = "full chunks (fp32 torch-CPU restatement; the reference ships no code for this model)"
    print(json.dumps({"impl": "reference", "metric": VLA_METRIC, "value": v, "unit": VLA_UNIT, "n_gpus": args.gpus, "steps": args.steps,
                      "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                      "dtype": "f32", "data": "synthetic", "config": vla_config_dict(c),
                      "cpu_baseline": {"value": v, "unit": VLA_UNIT, "cores": cores, "kind": "port", "sample": sample},
                      "e2e": {"value": v, "unit": VLA_UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}), flush=True)


def run_vla(args, rank, world, local_rank, *, steps, warmup, want_cpu, dist=None):
    import torch
    import cabi
    from oracle import smolvla          # synthetic weights / inputs (generators only) and the CPU baseline leg
    torch.cuda.set_device(local_rank)
    c = smolvla.VlaConfig()
    t_setup = time.perf_counter()
    w = smolvla.make_weights(c, seed=0)
    inp = smolvla.make_inputs(c, seed=rank)            # replicas: every rank its own request
    pol = cabi.VlaPolicy(c, device=local_rank)
    pol.load_weights(w)
    host = [t.contiguous().pin_memory() for t in (inp[0].float(), inp[1].int(), inp[2].float(), inp[3].float())]
    first = pol.chunk(*host)
    for _ in range(max(warmup, 3)):
        last = pol.chunk(*host)
    assert torch.equal(first, last), "graph replay differs from the kernel-by-kernel run"
    setup_s = time.perf_counter() - t_setup
    stream = torch.cuda.ExternalStream(pol.stream(), device=torch.device("cuda", local_rank))
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler = ClockSampler(local_rank)
    sampler.start()
    launches0 = pol.launch_count()[0]
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    e0.record(stream)
    for _ in range(steps):
        pol.enqueue()                                  # inputs resident on the device
    e1.record(stream)
    stream.synchronize()
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    dev_ms = e0.elapsed_time(e1)
    launches = pol.launch_count()[0] - launches0
    t0 = time.perf_counter()
    for _ in range(steps):
        out = pol.chunk(*host)                         # host buffers in, host actions out
    wall_s = time.perf_counter() - t0
    clocks = sampler.stop()
    pol.phase_ms()
    phases = pol.phase_ms()
    if dist is not None:
        t = torch.tensor([dev_ms, wall_s], dtype=torch.float64, device=torch.device("cuda", local_rank))
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dev_ms, wall_s = [float(x) for x in t.tolist()]
    fl = vla_flops(c)
    total = sum(fl.values())
    ms = dev_ms / steps
    peak_tf, kind = tensor_peak()
    achieved = total / (ms * 1e-3) / 1e12
    line = None
    if rank == 0:
        line = {"metric": VLA_METRIC, "value": world * steps / (dev_ms / 1e3), "unit": VLA_UNIT, "n_gpus": world, "steps": steps,
                "warmup": max(warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                "dtype": "bf16", "data": "synthetic",
                "config": dict(vla_config_dict(c), parallelism="single GPU" if world == 1 else f"{world} independent replicas"),
                "wall_s": wall_s, "setup_s": setup_s,
                "e2e": {"value": world * steps / wall_s, "unit": VLA_UNIT,
                        "h2d_bytes_per_step": sum(t.numel() * t.element_size() for t in host),
                        "d2h_bytes_per_step": out.numel() * 4, "api": "efm_b200_vla_chunk (C ABI, host buffers)"},
                "gpu_launches": launches, "clocks": clocks,
                "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak_tf, "unit": "TFLOP/s", "frac": achieved / peak_tf,
                             "traffic": None, "peak_kind": kind, "launch": "one chunk (one CUDA graph)",
                             "flops_per_launch": total, "flops_by_phase": fl, "us_per_launch": ms * 1e3,
                             "note": "the denoising loop (50-row GEMMs, 10 x 16 dependent layers) is latency-bound; only the "
                                     "vision tower and the prefix are tensor-bound"},
                "actions_head": [round(float(x), 4) for x in out[0, :4]]}
        line["roofline"]["phase_ms_kernel_by_kernel"] = {k: round(x, 3) for k, x in phases.items()}
        line["roofline"]["vision"] = tensor_report(fl["vision"], phases["vision"])
        if want_cpu:
            v, cores = vla_cpu_chunks_per_s(c, w, smolvla.make_inputs(c, seed=0), 2)
            line["cpu_baseline"] = {"value": v, "unit": VLA_UNIT, "cores": cores, "kind": "port",
                                    "sample": "2 full chunks (fp32 torch-CPU restatement)"}
    pol.close()
    return line


def summarise(line):
    """The per-configuration entry of the headline line."""
    if line is None:
        return None
    if line["metric"] == VLA_METRIC:
        return {"metric": VLA_METRIC, "value": line["value"], "unit": VLA_UNIT, "ms_per_chunk": line["ms_per_step"],
                "e2e": line["e2e"]["value"], "tensor_frac_whole_chunk": line["roofline"]["frac"],
                "vision_ms": line["roofline"]["vision"]["ms"], "vision_frac_of_bf16_peak": line["roofline"]["vision"]["frac_of_bf16_peak"],
                "phase_ms_kernel_by_kernel": line["roofline"]["phase_ms_kernel_by_kernel"], "workload": line["config"]["workload"]}
    out = {"metric": METRIC, "value": line["value"], "unit": UNIT, "decode_ms_per_token": line["decode_ms_per_token"],
           "hbm_frac": line["roofline"]["frac"], "hbm_frac_of_nominal_8tbs": line["roofline"]["frac_of_nominal_8tbs"],
           "prefill_ms": line["prefill_ms"], "prefill_frac_of_bf16_peak": line["prefill"]["frac_of_bf16_peak"],
           "ttft_ms": line["ttft_ms"], "e2e": line.get("e2e", {}).get("value"), "e2e_tokens_equal": line.get("e2e_tokens_equal"),
           "kernel_us": {k: v["us_per_launch"] for k, v in line["roofline"]["kernels"].items()},
           "steps": line["steps"], "workload": line["config"]["workload"], "weights": line["roofline"].get("weights", "bf16"),
           "bytes_per_decode_step": line["roofline"]["bytes_per_launch"]}
    if "vit" in line:
        out["vit_ms"] = line["vit_ms"]
        out["vit_frac_of_bf16_peak"] = line["vit"]["frac_of_bf16_peak"]
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", type=int, default=None, choices=[0, 1, 2, 3, 4],
                    help="run one configuration alone; default: configuration 3 (tensor parallel over the ranks) plus, on one GPU, "
                         "a short pass over the other four")
    ap.add_argument("--tokens", type=int, default=0, help="override the number of generated tokens")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-e2e", action="store_true", help="skip the public-API end-to-end leg (profiling runs)")
    ap.add_argument("--no-per-config", action="store_true", help="headline run without the pass over configurations 0, 1, 2, 4")
    ap.add_argument("--int4", action="store_true", help="one GPU: decode on a group-wise INT4 copy of the linears (C ABI only)")
    ap.add_argument("--tp-exchange", default="peer", choices=["peer", "nccl"],
                    help="config 3 on several GPUs: how the decode step sums the row-parallel partials")
    ap.add_argument("--prefill-attention", default="auto", choices=["auto", "bf16", "int8"],
                    help="auto: int8 for config 3 (as the benchmark specifies), bf16 otherwise")
    args = ap.parse_args()
    headline = args.config is None
    if headline:
        args.config = HEADLINE
    if args.prefill_attention == "auto":
        args.prefill_attention = "int8" if args.config == 3 else "bf16"
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else max(args.warmup, 1)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        if args.config == 4:
            run_vla_reference(args, rank)
        else:
            run_reference(args, rank)
        return
    if args.config == 3:
        line = run_tp(args, rank, world, local_rank)
        if headline and world == 1 and not args.no_per_config:
            per = {}
            for c in (0, 1, 2):
                per[str(c)] = summarise(run_text(args, c, 0, 1, local_rank, steps=2, warmup=3, want_cpu=False))
            per["1_int4"] = summarise(run_text(args, 1, 0, 1, local_rank, steps=2, warmup=3, want_cpu=False, int4=True))
            per["4"] = summarise(run_vla(args, 0, 1, local_rank, steps=5, warmup=3, want_cpu=False))
            if not args.int4:       # the headline workload once more with the decode pass on INT4 weights
                a4 = argparse.Namespace(**{**vars(args), "int4": True, "steps": 2, "no_e2e": True, "no_cpu": True})
                l4 = run_tp(a4, 0, 1, local_rank)
                per["3_int4"] = {"metric": METRIC, "value": l4["value"], "unit": UNIT, "decode_ms_per_token": l4["decode_ms_per_token"],
                                 "hbm_frac": l4["roofline"]["frac"], "prefill_ms": l4["prefill_ms"], "vit_ms": l4["vit_ms"],
                                 "ttft_ms": l4["ttft_ms"], "kernel_us": l4["roofline"].get("kernel_us_unoverlapped"), "steps": 2,
                                 "workload": l4["config"]["workload"], "weights": l4["roofline"]["weights"],
                                 "bytes_per_decode_step": l4["roofline"]["bytes_per_launch"], "tokens_head": l4["tokens_head"]}
            line["per_config"] = per
        if rank == 0:
            print(json.dumps(line), flush=True)
        return
    dist = None
    if world > 1:
        import torch
        import torch.distributed as dist_mod
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        torch.cuda.set_device(local_rank)
        dist = dist_mod
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank), timeout=datetime.timedelta(seconds=240))
    if args.config == 4:
        line = run_vla(args, rank, world, local_rank, steps=args.steps, warmup=args.warmup,
                       want_cpu=world == 1 and not args.no_cpu, dist=dist)
    else:
        line = run_text(args, args.config, rank, world, local_rank, steps=args.steps, warmup=args.warmup,
                        want_cpu=world == 1 and not args.no_cpu and not args.int4, dist=dist, int4=args.int4)
    if rank == 0:
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    try:
        main()
    except BaseException:
        # a failing rank must not linger in destructors that wait for its peers: report and leave at once, so that the
        # launcher ends the other ranks instead of letting them wait out a collective timeout
        import traceback
        traceback.print_exc()
        sys.stderr.flush()
        sys.stdout.flush()
        os._exit(1)
