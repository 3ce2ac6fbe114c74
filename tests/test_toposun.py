"""The Toposun decoder through the framework (configuration, loader, cache manager, step function,
scheduler, entry point) against the plain statement in tests/plain_toposun.py, on the host with the
stand-in kernels and on the GPU with the CUDA kernels, in 32-bit and in bfloat16.

Small configurations of their own and random weights: each mechanism alone, whole prompts against
token-by-token decoding, portions down to two tokens, mixed batches against each request alone, pages
and slots used again, positions at both edges of the window and of the kept first positions (in
prompts and decoded), the first tokens, long decoding, sizes that make mechanisms coincide (one head a
group, the whole head rotated, nothing kept, top 1, no shared expert, no feed-forward), and greedy
generation through the entry point."""
from __future__ import annotations

import json

import numpy as np
import pytest
import torch

import plain_kernels
import plain_toposun as T
import replay_cases as rc
from kvcore_b200 import (CacheConfig, DeviceConfig, KVCoreConfig, ModelConfig, SamplingParams, SchedulerConfig)
from kvcore_b200.config import ConfigError
from kvcore_b200.config.registry import model_spec_from_config
from kvcore_b200.engine.llm_engine import GenerationRequest, LLMEngine
from kvcore_b200.weights.safetensors_io import write_safetensors

BACKENDS = [pytest.param("cpu", id="host"), pytest.param("cuda:0", id="gpu", marks=pytest.mark.gpu)]
# largest |difference| of a row over the request's largest |logit|; in bfloat16 also the root mean square of a
# row's difference (its mean taken off) over that of the request's logits
TOLERANCE = {"float32": 3e-5, "bfloat16": 6e-2}
BF16_RMS_TOLERANCE = 3e-2


@pytest.fixture(params=BACKENDS)
def device(request, monkeypatch):
    if request.param == "cpu":
        plain_kernels.install(monkeypatch)
    return request.param


def attn(**kw):
    return T.attention_layer_config(**kw)


CONFIGS = {
    # a dense layer and a mixture layer with a shared expert; 2 heads a group, part of the head rotated
    "two_kinds": T.model_config([
        attn(heads=4, kv_heads=2, dim=16, window=8, keep_first=2, rot_dims=8, mlp=T.dense_mlp(48, limit=0.5)),
        attn(heads=4, kv_heads=2, dim=16, window=8, keep_first=2, rot_dims=8, mlp=T.moe_mlp(5, 2, 24, shared_ff=40)),
    ], vocab=96, width=32),
    # what the first makes unequal is equal here and the other way round: one head a group, the whole head
    # rotated, nothing kept, top 1 without a shared expert, a layer without feed-forward, other windows per layer
    "coincide": T.model_config([
        attn(heads=3, kv_heads=3, dim=32, window=20, keep_first=0, rot_dims=32, scale=0.3, mlp=None),
        attn(heads=3, kv_heads=3, dim=32, window=5, keep_first=7, rot_dims=2, base=50.0, mlp=T.moe_mlp(3, 1, 24)),
        attn(heads=2, kv_heads=1, dim=48, window=33, keep_first=1, rot_dims=0 + 16, mlp=T.moe_mlp(4, 4, 8, shared_ff=8)),
        # a head size and a turned part that no 16-byte vector fits, more kept positions than the window is long
        attn(heads=2, kv_heads=2, dim=20, window=9, keep_first=12, rot_dims=10, mlp=T.dense_mlp(24, limit=2.0)),
        attn(heads=4, kv_heads=1, dim=24, window=70, keep_first=3, rot_dims=12, mlp=T.moe_mlp(1, 1, 16)),
    ], vocab=61, width=40, eps=1e-6),
    # head sizes of the serving kernels (tensor-core prompt and decode kernels on the GPU), windows of
    # several pages, kept positions that end inside a page
    "serving_heads": T.model_config([
        attn(heads=4, kv_heads=1, dim=128, window=40, keep_first=5, rot_dims=64, mlp=T.dense_mlp(64, limit=1.0)),
        attn(heads=4, kv_heads=2, dim=64, window=24, keep_first=18, rot_dims=32, mlp=T.moe_mlp(6, 2, 32, shared_ff=16)),
    ], vocab=128, width=64),
}
LENGTHS = {"two_kinds": (1, 23, 45, 70, 37, 2), "coincide": (64, 1, 30, 90), "serving_heads": (150, 3, 97, 61)}


def write_folder(folder, cfg, seed):
    weights = T.random_weights(cfg, seed)
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(cfg))
    write_safetensors(folder / "model.safetensors", {k: v.to(torch.bfloat16) for k, v in weights.items()})
    return {k: v.double() for k, v in weights.items()}


@pytest.fixture(scope="module", params=list(CONFIGS))
def case(request, tmp_path_factory):
    name = request.param
    cfg = CONFIGS[name]
    folder = tmp_path_factory.mktemp(f"toposun_{name}")
    weights = write_folder(folder, cfg, seed=len(name))
    requests = {f"q{i}": rc.random_tokens(cfg["vocab"], n, 30 + i) for i, n in enumerate(LENGTHS[name])}
    reference, close_calls = {}, set()
    for rid, toks in requests.items():
        margins = []
        reference[rid] = T.forward(cfg, weights, toks, margins=margins).numpy()
        # positions where a router's choice hangs on less than bfloat16 keeps apart are not compared in bfloat16
        for gaps in margins:
            close_calls.update((rid, int(p)) for p in torch.nonzero(gaps < 2e-2).flatten())
    return dict(name=name, cfg=cfg, folder=folder, weights=weights, requests=requests, reference=reference,
                close_calls=close_calls)


def compare(rows, reference, dtype, close_calls=()):
    assert rows
    for (rid, pos), row in sorted(rows.items()):
        if dtype == "bfloat16" and (rid, pos) in close_calls:
            continue
        assert np.isfinite(row).all(), f"non-finite logits for {rid}@{pos}"
        err = np.abs(row - reference[rid][pos]).max() / np.abs(reference[rid]).max()
        assert err <= TOLERANCE[dtype], f"{rid}: first wrong position {pos} (error {err:.3e})"
        if dtype == "bfloat16":
            diff = row - reference[rid][pos]
            rms = np.sqrt(np.mean((diff - diff.mean()) ** 2)) / reference[rid].std()
            assert rms <= BF16_RMS_TOLERANCE, f"{rid}: first wrong position {pos} (rms error {rms:.3e})"


# ---- configuration -----------------------------------------------------------------------------------
def test_config_names_the_tensors_of_the_plain_statement():
    from kvcore_b200.parts.model import build_model

    for cfg in CONFIGS.values():
        spec = model_spec_from_config(cfg)
        assert spec.architecture == "Toposun"
        model = build_model(spec, dtype=torch.float32, device="meta")
        shapes = {slot.name: slot.shape for slot in model.weight_slots()}
        assert shapes == {k: tuple(v.shape) for k, v in T.random_weights(cfg, 0).items()}


def test_config_gives_every_constant_to_the_parts():
    cfg = CONFIGS["coincide"]
    spec = model_spec_from_config(cfg)
    mixer = spec.layers[1].mixer.params
    assert (mixer["sliding_window"], mixer["keep_first"], mixer["scale"]) == (5, 7, cfg["layers"][1]["mixer"]["scale"])
    assert mixer["position"].params["rotary_dim"] == 2 and mixer["position"].params["theta"] == 50.0
    assert mixer["qk_norm_eps"] == spec.final_norm.params["eps"] == 1e-6
    assert spec.layers[0].feed_forward is None and "feed_forward_norm" not in spec.layers[0].norms
    experts = spec.layers[2].feed_forward.params
    assert (experts["num_experts"], experts["top_k"], experts["expert_size"]) == (4, 4, 8)
    assert experts["shared"].params["intermediate_size"] == 8 and spec.layers[1].feed_forward.params["shared"] is None


@pytest.mark.parametrize("change,message", [
    (lambda c: c["layers"][0]["mixer"].update(vdim=8), "vdim"),
    (lambda c: c["layers"][0].update(type="recurrent"), "mixer of this design"),
    (lambda c: c["layers"][0]["mlp"].update(kind="conv"), "feed-forward of this design"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=9), "exceeds experts"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7), "even"),
    (lambda c: c["layers"][0]["mixer"].update(heads=3), "multiple"),
    (lambda c: c.pop("norm"), "norm"),
])
def test_config_refuses(change, message):
    cfg = json.loads(json.dumps(CONFIGS["two_kinds"]))
    change(cfg)
    with pytest.raises(ConfigError, match=message):
        model_spec_from_config(cfg)


def test_windowed_groups_keep_the_pages_of_the_kept_positions():
    """Layers with different (window, kept) pairs are cache groups of their own; a long request gives back
    the pages behind its window, never those that hold kept positions."""
    from kvcore_b200.cache.kv_manager import CacheGroupSpec, KVManager

    groups = [CacheGroupSpec(0, (0,), 2, 1, 8, window=5, keep_first=7), CacheGroupSpec(1, (1,), 2, 1, 8, window=5)]
    kv = KVManager(groups, num_pages=40, page_size=4, max_num_seqs=2, max_model_len=120)
    for step in range(30):
        assert kv.allocate_slots("a", 3)
        kv.advance("a", 3)
        kv.check_invariants()
    kept, plain = kv.block_ids("a")
    first_visible = 90 - 5 + 1
    assert all(page != 0 for page in kept[:2]) and all(page == 0 for page in kept[2: first_visible // 4])
    assert all(page == 0 for page in plain[: first_visible // 4])
    assert all(page != 0 for page in kept[first_visible // 4:]) and all(page != 0 for page in plain[first_visible // 4:])
    kv.free("a")
    kv.check_invariants()
    assert kv.num_free_pages() == [39, 39]


# ---- the cuttings ---------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_cuttings_match_the_plain_statement(case, dtype, device, tmp_path):
    cfg, requests = case["cfg"], case["requests"]
    traces = {
        "whole": rc.trace_whole(requests),
        "tail": rc.trace_decode_tail(requests, tail=40),                  # the window passes over decoded tokens
        "chunks": rc.trace_chunks(requests, sizes=(7, 3, 16, 2, 5, 1, 9, 2, 31)),
        "mixed": rc.trace_mixed(requests, max_live=4, seed=3),
    }
    results = {}
    for name, steps in traces.items():
        out = tmp_path / name
        rc.run_inprocess(case["folder"], dtype, steps, out, rc.peak_tokens(steps), device=device,
                         fill_freed_pages="poison" if name == "mixed" else None)
        rows = rc.collect(steps, out, cfg["vocab"])
        assert len(rows) == sum(len(t) for t in requests.values())
        compare(rows, case["reference"], dtype, case["close_calls"])
        results[name] = rows
    if dtype == "float32" and device != "cpu":
        # every kernel of the 32-bit path sums in an order that depends on the position only
        for name in ("tail", "chunks", "mixed"):
            for key, row in results["whole"].items():
                assert np.array_equal(row, results[name][key]), f"{name} differs from whole at {key}"


def test_residual_stream_after_every_layer(case, device):
    """Layer by layer: the 32-bit stream after each block against the plain statement's."""
    from kvcore_b200.engine.trace_replay import build_replay
    from kvcore_b200.engine.step import StepEntry

    tokens = case["requests"]["q1"]
    step_function, kv = build_replay(str(case["folder"]), "float32", 256, device=device)
    model = step_function.model
    seen = []
    for block in model.blocks:
        original = block.forward

        def recording(h, residual, ctx, cache, original=original):
            out = original(h, residual, ctx, cache)
            seen.append(out[1].detach().clone().cpu())
            return out
        block.forward = recording
    assert kv.allocate_slots("x", len(tokens))
    step_function.step([StepEntry("x", tokens, [len(tokens) - 1])])
    collected = []
    T.forward(case["cfg"], case["weights"], tokens, collected)
    assert len(seen) == len(collected)
    for index, (got, want) in enumerate(zip(seen, collected)):
        assert got.dtype == torch.float32
        torch.testing.assert_close(got.double(), want, rtol=2e-5, atol=2e-5, msg=lambda m: f"layer {index}: {m}")


def test_pages_and_slots_are_used_again(case, device, tmp_path):
    """A pool for the largest live set only: the mixed trace needs more pages over its life than the pool
    has, and more requests than slots in a row."""
    requests = dict(case["requests"])
    requests.update({f"again{i}": toks for i, toks in enumerate(case["requests"].values())})
    steps = rc.trace_mixed(requests, max_live=3, seed=11)
    peak = rc.peak_tokens(steps)
    assert sum(-(-len(t) // 16) * 16 for t in requests.values()) > peak
    out = tmp_path / "o"
    step_function, kv = rc.run_inprocess(case["folder"], "float32", steps, out, peak, device=device,
                                         fill_freed_pages="poison")
    assert all(pool.num_free == pool.num_usable for pool in kv.pools)
    reference = dict(case["reference"])
    reference.update({f"again{i}": ref for i, ref in enumerate(case["reference"].values())})
    compare(rc.collect(steps, out, case["cfg"]["vocab"]), reference, "float32")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_past_windows_and_pages(dtype, device, tmp_path):
    """Two prompt tokens, then two hundred single tokens: every window passes over decoded tokens, pages
    behind the windows go back to the pool while the request lives, the kept positions stay."""
    cfg = CONFIGS["serving_heads"] if device != "cpu" else CONFIGS["two_kinds"]
    folder = tmp_path / "m"
    weights = write_folder(folder, cfg, seed=5)
    tokens = rc.random_tokens(cfg["vocab"], 200, 77)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": tokens[:2], "want": [0, 1]}], "end": []}]
    for pos in range(2, len(tokens)):
        steps.append({"step": pos - 1, "entries": [{"id": "a", "tokens": [tokens[pos]], "want": [0]}],
                      "end": ["a"] if pos == len(tokens) - 1 else []})
    out = tmp_path / "o"
    # a pool of 7 pages of 16 tokens: fewer than the request would take without its windows
    from kvcore_b200.engine.trace_replay import build_replay

    step_function, kv = build_replay(str(folder), dtype, 112, device=device, fill_freed_pages="poison", max_model_len=256)
    rc.run_on(step_function, kv, steps, out)
    margins = []
    reference = {"a": T.forward(cfg, weights, tokens, margins=margins).numpy()}
    close_calls = {("a", int(p)) for gaps in margins for p in torch.nonzero(gaps < 2e-2).flatten()}
    compare(rc.collect(steps, out, cfg["vocab"]), reference, dtype, close_calls)


def test_each_mechanism_changes_the_logits(tmp_path):
    """The plain statement itself: leaving a mechanism out moves the logits by far more than any tolerance
    here, so a test that passes has seen it.  (Guards the tests, not the product.)"""
    cfg = CONFIGS["two_kinds"]
    weights = T.random_weights(cfg, 9, dtype=torch.float64)
    tokens = rc.random_tokens(cfg["vocab"], 40, 3)
    base = T.forward(cfg, weights, tokens)

    def moved(change):
        other = json.loads(json.dumps(cfg))
        change(other)
        return float((T.forward(other, weights, tokens) - base).abs().max() / base.abs().max())

    assert moved(lambda c: [l["mixer"]["mask"].update(keep_first=0) for l in c["layers"]]) > 1e-3
    assert moved(lambda c: [l["mixer"]["mask"].update(size=9) for l in c["layers"]]) > 1e-3
    assert moved(lambda c: [l["mixer"]["rot"].update(dims=16) for l in c["layers"]]) > 1e-3
    assert moved(lambda c: c["layers"][0]["mlp"].update(limit=5.0)) > 1e-3
    assert moved(lambda c: c["layers"][1]["mlp"]["router"].update(top=1)) > 1e-3
    assert moved(lambda c: c["layers"][1]["mlp"].pop("shared")) > 1e-3


# ---- the entry point and the scheduler -------------------------------------------------------------------
def plain_greedy(cfg, weights, prompt, steps):
    tokens = list(prompt)
    for _ in range(steps):
        tokens.append(int(T.forward(cfg, weights, tokens)[-1].argmax()))
    return tokens[len(prompt):]


@pytest.mark.parametrize("name,budget", [("two_kinds", 16), ("coincide", 7)])
def test_greedy_generation_through_the_entry_point(device, tmp_path, name, budget):
    cfg = CONFIGS[name]
    folder = tmp_path / "m"
    weights = write_folder(folder, cfg, seed=21)
    prompts = [rc.random_tokens(cfg["vocab"], n, 60 + i) for i, n in enumerate((5, 19, 33))]
    config = KVCoreConfig(
        model_config=ModelConfig(model=str(folder), dtype="float32", max_model_len=128),
        cache_config=CacheConfig(block_size=16, num_gpu_blocks=24),
        scheduler_config=SchedulerConfig(max_num_seqs=4, max_num_scheduled_tokens=budget,
                                         max_num_partial_prefills=4, max_long_partial_prefills=4),
        device_config=DeviceConfig(device=device),
    )
    engine = LLMEngine(config)
    requests = [GenerationRequest(f"g{i}", SamplingParams(max_tokens=12, temperature=0.0), tuple(p))
                for i, p in enumerate(prompts)]
    outputs = engine.generate(requests)
    for prompt, output in zip(prompts, outputs):
        assert list(output.output_token_ids) == plain_greedy(cfg, weights, prompt, 12)
    kv = engine.engine_core.model_runner.kv_manager
    kv.check_invariants()
    assert not kv.live_requests()


# ---- the programs, each in a process of its own ------------------------------------------------------------
@pytest.mark.gpu
def test_offline_batch_program_on_a_toposun_folder(tmp_path):
    import ast
    import re
    import subprocess
    import sys

    cfg = CONFIGS["serving_heads"]
    folder = tmp_path / "m"
    weights = write_folder(folder, cfg, seed=4)
    prompts = {f"req-{i}": rc.random_tokens(cfg["vocab"], n, 80 + i) for i, n in enumerate((70, 9, 33))}
    (tmp_path / "requests.json").write_text(json.dumps(
        [dict(request_id=rid, prompt_token_ids=tokens) for rid, tokens in prompts.items()]))
    command = [sys.executable, str(rc.ROOT / "bin" / "kvcore_offline_batch"), "--model", str(folder), "--dtype", "float32",
               "--prompt-tokens-file", str(tmp_path / "requests.json"), "--max-tokens", "6", "--block-size", "16",
               "--num-gpu-blocks", "64", "--max-model-len", "256", "--max-num-seqs", "4",
               "--max-num-scheduled-tokens", "48", "--max-num-partial-prefills", "4", "--max-long-partial-prefills", "4",
               "--log-level", "WARNING"]
    result = subprocess.run(command, capture_output=True, text=True, timeout=300)
    assert result.returncode == 0, result.stderr[-2000:]
    found = {m["id"]: list(ast.literal_eval(m["ids"])) for m in re.finditer(
        r"^\[(?P<id>[^\]]+)\] finish_reason=\S+\ntoken_ids=(?P<ids>\(.*\))$", result.stdout, re.M)}
    assert list(found) == list(prompts)
    for rid, prompt in prompts.items():
        assert found[rid] == plain_greedy(cfg, weights, prompt, 6)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_program_on_a_toposun_folder(case, dtype, tmp_path):
    """``bin/trace_run`` as a user drives it: a step, its ``done`` line, the next step."""
    if case["name"] != "serving_heads":
        pytest.skip("one configuration is enough for the subprocess run")
    steps = rc.trace_mixed(case["requests"], max_live=3, seed=5)
    steps.insert(1, {"step": 1000, "entries": [], "end": []})      # a step that brings nothing
    out = tmp_path / "out"
    rc.run_subprocess(case["folder"], dtype, steps, out, rc.peak_tokens(steps))
    rows = rc.collect(steps, out, case["cfg"]["vocab"])
    assert len(rows) == sum(len(t) for t in case["requests"].values())
    compare(rows, case["reference"], dtype, case["close_calls"])
