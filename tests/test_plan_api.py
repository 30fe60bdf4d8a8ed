"""EdgeFM.plan() for task = trajectory_planning (action-chunk policy): configuration errors on any machine, parity with
oracle/smolvla.py through the public Python API on a GPU.  Mirrors the request / response contract of the reference's
planner tests (tests/engine/test_planner_policy_api.py: plan(request_id, {name: Tensor}) -> {"trajectory": Tensor})."""
import ctypes
import json
import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "edge-fm-x_b200", "python"))

from oracle import smolvla  # noqa: E402

TOL = 3e-2


def _write_policy(tmp_path, cfg, weights, planner, task="trajectory_planning"):
    from safetensors.torch import save_file
    model_dir = tmp_path / "policy"
    model_dir.mkdir()
    fields = ("image_size patch vit_layers vit_hidden vit_heads vit_mlp shuffle n_images hidden layers q_heads kv_heads head_dim "
              "mlp vocab lang_tokens expert_hidden expert_mlp state_dim action_dim chunk steps rope_theta rms_eps ln_eps").split()
    (model_dir / "config.json").write_text(json.dumps({k: getattr(cfg, k) for k in fields}))
    if weights is not None:
        save_file({k: v.contiguous() for k, v in weights.items()}, str(model_dir / "model.safetensors"))
    engine = {"task": task, "model_name": "smolvla", "prefill_model_path": str(model_dir),
              "runtime": {"device": "cuda", "device_id": 0}, "planner": planner}
    path = tmp_path / "engine.json"
    path.write_text(json.dumps(engine))
    return str(path)


def _tensor(edge_fm, t):
    dt = {torch.float32: edge_fm.DType.Float32, torch.int32: edge_fm.DType.Int32}[t.dtype]
    return edge_fm.Tensor(t.data_ptr(), list(t.shape), dt, edge_fm.Device.CPU)


def _values(t, n):
    return torch.tensor((ctypes.c_float * n).from_address(t.data_ptr())[:])


def test_unsupported_planner_settings_are_configuration_errors(tmp_path):
    import edge_fm
    cfg = smolvla.VlaConfig.tiny()
    for i, planner in enumerate(({"type": "candidate_scoring"}, {"type": "iterative_denoise", "sampler": "ddim"})):
        d = tmp_path / f"case{i}"
        d.mkdir()
        with pytest.raises(ValueError):
            edge_fm.EdgeFM(_write_policy(d, cfg, None, planner))
    d = tmp_path / "inferred"           # no task key: the policy model name selects the planner task
    d.mkdir()
    path = _write_policy(d, cfg, None, {"type": "candidate_scoring"})
    doc = json.loads(open(path).read())
    del doc["task"]
    open(path, "w").write(json.dumps(doc))
    with pytest.raises(ValueError, match="planner.type"):
        edge_fm.EdgeFM(path)
    d = tmp_path / "task"
    d.mkdir()
    with pytest.raises(ValueError, match="Unsupported task"):
        edge_fm.EdgeFM(_write_policy(d, cfg, None, {}, task="speech"))


@pytest.mark.gpu
def test_plan_equals_oracle_and_reports_metrics(tmp_path):
    import edge_fm
    cfg = smolvla.VlaConfig.tiny()
    w = smolvla.make_weights(cfg, seed=31)
    images, ids, state, noise = smolvla.make_inputs(cfg, seed=31)
    eng = edge_fm.EdgeFM(_write_policy(tmp_path, cfg, w, {"type": "iterative_denoise", "sampler": "euler_flow",
                                                          "num_steps": cfg.steps, "output_tensor": "actions",
                                                          "trajectory_shape": [cfg.chunk, cfg.action_dim], "seed": 5}))
    held = [images.contiguous(), ids.contiguous(), state.contiguous(), noise.contiguous()]
    inputs = {"images": _tensor(edge_fm, held[0]), "lang_tokens": _tensor(edge_fm, held[1]), "state": _tensor(edge_fm, held[2]),
              "current_actions": _tensor(edge_fm, held[3])}
    out = eng.plan(0, inputs)
    assert sorted(out) == ["actions", "trajectory"]
    assert out["trajectory"].shape() == [cfg.chunk, cfg.action_dim]
    got = _values(out["trajectory"], cfg.chunk * cfg.action_dim).reshape(cfg.chunk, cfg.action_dim)
    want = smolvla.VlaOracle(cfg, w, mode="bf16_points").chunk(images, ids, state, noise)
    assert (got - want).abs().max().item() < TOL
    m = eng.last_plan_metrics()
    assert m["plan_steps"] == cfg.steps and m["stage_calls"] == cfg.steps + 1 and m["plan_ms"] > 0
    # without the state tensor the start is drawn from planner.trajectory_shape / seed: deterministic
    del inputs["current_actions"]
    a = _values(eng.plan(0, inputs)["trajectory"], cfg.chunk * cfg.action_dim)
    b = _values(eng.plan(0, inputs)["trajectory"], cfg.chunk * cfg.action_dim)
    assert torch.equal(a, b) and torch.isfinite(a).all()
    with pytest.raises(ValueError):
        eng.plan(0, {"images": inputs["images"]})
    with pytest.raises(ValueError):
        eng.generate(edge_fm.Request(0, [1, 2, 3]))
