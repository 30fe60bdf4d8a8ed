"""CPU: the compact-vocabulary contract of the generate() boundary (edge_fm::CompactVocab), driven through a
small C++ program linked against the in-tree host engine.  Cases follow the reference's own list
(tests/cpp/test_compact_vocab.cpp: remap/restore, disabled no-op, unknown ids, mapping shape, kept special /
stop / EOS ids) plus the pre-pruned checkpoint check and the embedding-placeholder rule of
doc/compact_vocab_contract.md."""
import importlib.util
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "edge-fm-x_b200")


@pytest.fixture(scope="module")
def driver(tmp_path_factory):
    lib = os.path.join(PKG, "lib", "libedge_fm.so")
    if not os.path.exists(lib):
        pytest.fail("libedge_fm.so is missing: run python edge-fm-x_b200/build.py")
    sys.path.insert(0, PKG)
    spec = importlib.util.spec_from_file_location("efm_build", os.path.join(PKG, "build.py"))
    build = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(build)
    exe = str(tmp_path_factory.mktemp("cv") / "compact_vocab_check")
    cmd = ["g++", "-O1", "-std=c++17", os.path.join(ROOT, "tests", "cpp", "compact_vocab_check.cpp"), "-o", exe,
           "-I", os.path.join(PKG, "src", "engine"), "-I", os.path.join(PKG, "include"), "-I", os.path.join(ROOT, "include"),
           "-I", build.dlpack_include(), "-L", os.path.join(PKG, "lib"), "-ledge_fm", "-lefm_b200", "-Wl,-rpath," + os.path.join(PKG, "lib"),
           "-Wl,-rpath,/usr/local/cuda/lib64"]
    subprocess.run(cmd, check=True, capture_output=True, text=True)
    return exe


def make_deployment(tmp_path, *, mapping=None, enabled=True, vocab_size=None, eos=None, stop=None, cv_extra=None):
    """Engine JSON + model dir (config.json only: CompactVocab never opens the weights) + mapping file."""
    base = dict(format="edgefm.compact_vocab.v1", original_vocab_size=8, compact_vocab_size=4,
                old_to_new=[0, -1, 1, -1, 2, -1, -1, 3], new_to_old=[0, 2, 4, 7], special_token_ids=[7])
    if mapping:
        base.update(mapping)
    model = tmp_path / "model"
    model.mkdir(exist_ok=True)
    cfg = dict(vocab_size=vocab_size if vocab_size is not None else base["compact_vocab_size"], hidden_size=64,
               num_hidden_layers=1, num_attention_heads=1, num_key_value_heads=1, intermediate_size=64)
    if eos is not None:
        cfg["eos_token_id"] = eos
    (model / "config.json").write_text(json.dumps(cfg))
    (tmp_path / "map.json").write_text(json.dumps(base))
    cv = dict(enabled=enabled, mapping_path="map.json", reject_unknown_input_ids=True)
    if cv_extra:
        cv.update(cv_extra)
    eng = dict(model_name="Qwen2.5", prefill_model_path=str(model), compact_vocab=cv,
               sampling=dict(stop_token_ids=stop or []))
    path = tmp_path / "engine.json"
    path.write_text(json.dumps(eng))
    return str(path)


def run(driver, cfg, op, *ids):
    out = subprocess.run([driver, cfg, op, *[str(i) for i in ids]], capture_output=True, text=True, check=True).stdout.split()
    return out[0], out[1:]


def test_non_identity_remap_and_restore(driver, tmp_path):
    cfg = make_deployment(tmp_path)
    assert run(driver, cfg, "info") == ("ok", ["1", "8", "4"])
    assert run(driver, cfg, "remap", 7, 0, 4, 2) == ("ok", ["3", "0", "2", "1"])
    assert run(driver, cfg, "restore", 3, 0, 2, 1) == ("ok", ["7", "0", "4", "2"])


def test_disabled_is_the_identity(driver, tmp_path):
    cfg = make_deployment(tmp_path, enabled=False, vocab_size=8)
    assert run(driver, cfg, "info")[1][0] == "0"
    assert run(driver, cfg, "remap", 5, 1, 1000) == ("ok", ["5", "1", "1000"])
    assert run(driver, cfg, "restore", 6) == ("ok", ["6"])


def test_pruned_or_out_of_range_request_ids_are_refused(driver, tmp_path):
    cfg = make_deployment(tmp_path)
    for bad in (1, 8, -1):
        st, rest = run(driver, cfg, "remap", 0, bad)
        assert st == "error" and rest[0] == "InvalidRequestError" and "absent" in " ".join(rest)
    st, rest = run(driver, cfg, "required", 3)                 # a deployment id: configuration problem
    assert st == "error" and rest[0] == "ConfigurationError"
    st, rest = run(driver, cfg, "restore", 4)                  # the model can not produce this
    assert st == "error" and rest[0] == "InternalError"


@pytest.mark.parametrize("mapping,needle", [
    (dict(format="something.else"), "format"),
    (dict(old_to_new=[0, -1, 1]), "old_to_new length"),
    (dict(new_to_old=[0, 2, 4]), "new_to_old length"),
    (dict(new_to_old=[0, 2, 4, 6]), "disagree"),
    (dict(old_to_new=[0, -1, 1, -1, 2, -1, 3, 3]), "disagree"),
    (dict(old_to_new=[0, -1, 1, -1, 2, -1, -1, 9]), "out-of-range"),
    (dict(compact_vocab_size=9), "<= original_vocab_size"),
    (dict(original_vocab_size=0), "positive"),
])
def test_mapping_shape_validation(driver, tmp_path, mapping, needle):
    st, rest = run(driver, make_deployment(tmp_path, mapping=mapping, vocab_size=4), "info")
    assert st == "error" and rest[0] == "ConfigurationError" and needle in " ".join(rest)


def test_special_stop_and_eos_ids_must_survive(driver, tmp_path):
    st, rest = run(driver, make_deployment(tmp_path, mapping=dict(special_token_ids=[5])), "info")
    assert st == "error" and "special_token_ids" in " ".join(rest)
    st, rest = run(driver, make_deployment(tmp_path, stop=[3]), "info")
    assert st == "error" and "stop_token_ids" in " ".join(rest)
    st, rest = run(driver, make_deployment(tmp_path, eos=6), "info")
    assert st == "error" and "eos" in " ".join(rest)
    assert run(driver, make_deployment(tmp_path, eos=4, stop=[2]), "info")[0] == "ok"


def test_checkpoint_must_be_pre_pruned_and_unknown_fallback_is_refused(driver, tmp_path):
    st, rest = run(driver, make_deployment(tmp_path, vocab_size=8), "info")
    assert st == "error" and "pre-pruned" in " ".join(rest)
    st, rest = run(driver, make_deployment(tmp_path, cv_extra=dict(reject_unknown_input_ids=False)), "info")
    assert st == "error" and "reject_unknown_input_ids" in " ".join(rest)
    st, rest = run(driver, make_deployment(tmp_path, cv_extra=dict(mapping_path="missing.json")), "info")
    assert st == "error" and "Cannot open" in " ".join(rest)


def test_embedding_placeholders_must_stay_contiguous(driver, tmp_path):
    m = dict(original_vocab_size=8, compact_vocab_size=5, old_to_new=[0, -1, 1, 2, 3, -1, -1, 4], new_to_old=[0, 2, 3, 4, 7])
    cfg = make_deployment(tmp_path, mapping=m)
    assert run(driver, cfg, "embed", 2, 3) == ("ok", ["1"])            # 2,3,4 -> 1,2,3
    st, rest = run(driver, cfg, "embed", 4, 2)                          # 4 -> 3 but 5 is pruned
    assert st == "error" and rest[0] == "InvalidRequestError"
    st, rest = run(driver, cfg, "embed", 0, 2)                          # 0 -> 0 but 1 is pruned
    assert st == "error"
    m2 = dict(original_vocab_size=4, compact_vocab_size=3, old_to_new=[2, 0, 1, -1], new_to_old=[1, 2, 0], special_token_ids=[0])
    cfg2 = make_deployment(tmp_path, mapping=m2)
    st, rest = run(driver, cfg2, "embed", 0, 2)                         # kept, but 0,1 -> 2,0: not contiguous
    assert st == "error" and "contiguous" in " ".join(rest)
    assert run(driver, cfg2, "embed", -1, 5) == ("ok", ["-1"])
