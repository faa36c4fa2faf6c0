"""The example scripts run end to end on CPU ranks (gloo), with and without on-demand communication."""
import json
import os
import subprocess
import sys

import pytest

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port() -> int:
    import socket
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("env", [{"ODC": "1"}, {"ODC": "1", "HPZ": "1"}, {"ODC": "0"}])
def test_fsdp2_example_cpu(env, tmp_path):
    e = dict(os.environ, **env, ODC_SYMMETRIC_SIZE="256M")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", str(_free_port()),
           os.path.join(REPO, "examples/FSDP2/example.py"), "--cpu", "--checkpoint-dir", str(tmp_path)]
    r = subprocess.run(cmd, env=e, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    assert "step 9 loss" in r.stdout


@pytest.mark.parametrize("script,env,packing,extra", [
    ("train_fsdp2.py", {"ODC": "1"}, "DynamicDiffMicro", ["--save-hf-checkpoint", "{tmp}/hf_out"]),  # unequal microbatch counts
    ("train_fsdp2.py", {"ODC": "0", "ODC_DEBUG_PACKING": "1", "ODC_WANDB": "1", "WANDB_MODE": "disabled"}, "DynamicSameMicro", []),  # lock-step baseline
    ("train_fsdp1.py", {"ODC": "1"}, "DynamicDiffMicro", ["--loss-head", "logprobs"]),   # per-token log-prob head
    ("train_fsdp2.py", {"ENGINE": "fused"}, "DynamicDiffMicro", []),   # the fused-kernel decoder engine
])
def test_llm_trainers_cpu(script, env, packing, extra, tmp_path):
    e = dict(os.environ, **env, ODC_SYMMETRIC_SIZE="256M", ODC_OUT_DIR=str(tmp_path))
    port = _free_port()
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", str(port), os.path.join(REPO, "examples/llm_training", script), "--cpu",
           "--model_name", "tiny", "--steps", "2", "--minibatch_size", "4", "--num-sequences", "32",
           "--length-dist", "uniform", "--limit_dataset_token_len", "200", "--max_token_len", "512",
           "--packing_method", packing, "--run_name", "cpu_smoke"] + [x.replace("{tmp}", str(tmp_path)) for x in extra]
    r = subprocess.run(cmd, env=e, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    lines = [json.loads(l) for l in r.stdout.splitlines() if l.startswith("{")]
    assert [l["step"] for l in lines] == [0, 1]
    assert all(l["loss"] == l["loss"] and l["tokens"] > 0 for l in lines)
    assert (tmp_path / "cpu_smoke.done").exists()
    if "--save-hf-checkpoint" in extra:   # FSDP2 shards gathered into a Hugging Face checkpoint folder by rank 0
        sys.path.insert(0, REPO)
        from odc_b200.models import get_config
        from odc_b200.models.hf import load_hf_checkpoint
        cfg, sd = load_hf_checkpoint(str(tmp_path / "hf_out"))
        assert cfg == get_config("tiny") and tuple(sd["layers.1.mlp.w_down"].shape) == (cfg.hidden_size, cfg.intermediate_size)
    if env.get("ODC_DEBUG_PACKING") == "1":   # every rank's microbatch composition, printed by rank 0
        assert "rank 0 " in r.stdout and "rank 1 " in r.stdout


@pytest.mark.parametrize("script", ["all_gather.py", "reduce_scatter.py"])
def test_primitive_benchmarks_cpu(script, tmp_path):
    """The two micro-benchmarks check their result against the library collective; run them small on CPU ranks."""
    _run_prim_bench(script, tmp_path, [])


def test_gather_random_subsets_cpu(tmp_path):
    """``all_gather.py --peers=random``: every rank pulls random subsets of its peers (3 CPU ranks)."""
    _run_prim_bench("all_gather.py", tmp_path, ["--peers=random"], world=3)


def _run_prim_bench(script, tmp_path, extra, world=2):
    e = dict(os.environ, ODC_BENCH_CPU="1", ODC_SYMMETRIC_SIZE="64M", ODC_OUT_DIR=str(tmp_path))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(world), "--master-addr",
           "127.0.0.1", "--master-port", str(_free_port()), os.path.join(REPO, "examples", script),
           "--size-min=4096", "--size-max=65536"] + extra
    r = subprocess.run(cmd, env=e, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    out = [f for f in os.listdir(tmp_path) if f.endswith(".json")]
    assert len(out) == 1
    rows = json.load(open(tmp_path / out[0]))
    assert [row["shard_bytes"] for row in rows] == [4096, 8192, 16384, 32768, 65536]


def test_bench_reference_arm_reports_one_json_line():
    """``bench.py --impl reference`` either runs the reference or prints why it cannot, as one JSON line, exit code 0
    (no GPU is needed to get as far as the reference's import)."""
    r = subprocess.run([sys.executable, os.path.join(REPO, "bench.py"), "--impl", "reference", "--gpus", "1", "--steps", "1",
                        "--warmup", "1"], capture_output=True, text=True, timeout=600,
                       env=dict(os.environ, RANK="0", WORLD_SIZE="1"))
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [json.loads(l) for l in r.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1 and lines[0]["impl"] == "reference"
    assert "unavailable" in lines[0] or {"metric", "value", "n_gpus"} <= set(lines[0])
    # a rank other than 0 prints nothing: the driver reads one line per job
    r1 = subprocess.run([sys.executable, os.path.join(REPO, "bench.py"), "--impl", "reference", "--gpus", "2"],
                        capture_output=True, text=True, timeout=600, env=dict(os.environ, RANK="1", WORLD_SIZE="2"))
    if "unavailable" in lines[0]:
        assert r1.returncode == 0 and not [l for l in r1.stdout.splitlines() if l.startswith("{")]


@pytest.mark.parametrize("script,env", [("train_fsdp2.py", {"ENGINE": "fused"}), ("train_fsdp1.py", {"ODC": "1"})])
def test_trainers_start_from_a_hugging_face_checkpoint(script, env, tmp_path):
    """``--hf-checkpoint``: architecture and initial weights come from a checkpoint folder (written here in the
    Hugging Face layout from a tiny Qwen2-style decoder), not from a preset and a seed."""
    import torch
    sys.path.insert(0, REPO)
    from odc_b200.models import DecoderLM, get_config
    from odc_b200.models.hf import save_hf_checkpoint
    cfg = get_config("tiny", qkv_bias=True, tie_embeddings=True, vocab_size=512)
    src = DecoderLM(cfg)
    src.reset_parameters(seed=3)
    ckpt = tmp_path / "ckpt"
    save_hf_checkpoint(str(ckpt), src.state_dict(), cfg, dtype=torch.float32)
    e = dict(os.environ, **env, ODC_SYMMETRIC_SIZE="256M", ODC_OUT_DIR=str(tmp_path))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", str(_free_port()), os.path.join(REPO, "examples/llm_training", script), "--cpu",
           "--hf-checkpoint", str(ckpt), "--steps", "1", "--minibatch_size", "4", "--num-sequences", "16",
           "--length-dist", "uniform", "--limit_dataset_token_len", "200", "--max_token_len", "512",
           "--run_name", "from_hf", "--save-hf-checkpoint", str(tmp_path / "out")]
    r = subprocess.run(cmd, env=e, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    lines = [json.loads(l) for l in r.stdout.splitlines() if l.startswith("{")]
    # the trained model was written back in the same layout: same architecture, same names, moved weights
    from odc_b200.models.hf import load_hf_checkpoint
    cfg2, sd2 = load_hf_checkpoint(str(tmp_path / "out"))
    assert cfg2 == cfg and set(sd2) == set(src.state_dict())
    moved = (sd2["layers.0.attn.wqkv"].float() - src.state_dict()["layers.0.attn.wqkv"]).abs().max()
    assert 0 < float(moved) < 0.1
    # the default --model_name is a 1.5B preset: finishing at all means the checkpoint's tiny architecture was used;
    # near-uniform predictions over its 512 words bound the (sequence-count weighted) loss by ln(512) = 6.24
    assert len(lines) == 1 and 0.0 < lines[0]["loss"] < 6.5 and lines[0]["tokens"] > 0, lines


@pytest.mark.parametrize("env", [{"ODC": "1"}])
def test_trainer_resumes_from_its_checkpoint(env, tmp_path):
    """Two minibatches, stop, start again with ``--steps 3``: the job runs only the third minibatch, from the saved
    model, optimizer state and step, and its loss is the one an uninterrupted run sees.  (FSDP2 patch + FusedAdamW
    here; the fused engine resumes in the launcher test below, and its state round trip is compared tensor by tensor in
    test_fused_engine_cpu.py.)"""
    def run(steps, ckpt):
        e = dict(os.environ, **env, ODC_SYMMETRIC_SIZE="256M", ODC_OUT_DIR=str(tmp_path))
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
               "127.0.0.1", "--master-port", str(_free_port()), os.path.join(REPO, "examples/llm_training/train_fsdp2.py"),
               "--cpu", "--model_name", "tiny", "--steps", str(steps), "--minibatch_size", "4", "--num-sequences", "32",
               "--length-dist", "uniform", "--limit_dataset_token_len", "200", "--max_token_len", "512", "--lr", "1e-3",
               "--run_name", "resume"] + (["--checkpoint-dir", str(ckpt), "--checkpoint-every", "1"] if ckpt else [])
        r = subprocess.run(cmd, env=e, capture_output=True, text=True, timeout=600)
        assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
        return {l["step"]: l["loss"] for l in (json.loads(x) for x in r.stdout.splitlines() if x.startswith("{"))}

    whole = run(3, None)
    first = run(2, tmp_path / "ck")
    second = run(3, tmp_path / "ck")
    assert sorted(whole) == [0, 1, 2] and sorted(first) == [0, 1] and sorted(second) == [2]
    assert first[1] == pytest.approx(whole[1], rel=1e-4)
    assert second[2] == pytest.approx(whole[2], rel=1e-3)
    assert second[2] != pytest.approx(whole[0], rel=1e-3)   # not a fresh start


def test_launcher_restarts_a_failed_job_which_resumes(tmp_path):
    """The failure drill end to end.  A rank leaves between minibatches (made on the host); the other reports it and
    exits with the temporary-failure code instead of waiting; ``MAX_RESTARTS=1 bash launch.sh ...`` starts all ranks
    again, and the second attempt resumes from the checkpoint and completes."""
    e = dict(os.environ, ENGINE="fused", ODC_SYMMETRIC_SIZE="256M", ODC_OUT_DIR=str(tmp_path), ODC_HEARTBEAT_S="30",
             ODC_WAIT_TIMEOUT_MS="20000", ODC_INJECT_LEAVE="1:1", MAX_RESTARTS="1", GPUS_PER_NODE="2",
             MASTER_PORT=str(_free_port()))
    cmd = ["bash", os.path.join(REPO, "launch.sh"), os.path.join(REPO, "examples/llm_training/train_fsdp2.py"),
           "--cpu", "--model_name", "tiny", "--steps", "3", "--minibatch_size", "4", "--num-sequences", "32",
           "--length-dist", "uniform", "--limit_dataset_token_len", "200", "--max_token_len", "512",
           "--run_name", "restart", "--checkpoint-dir", str(tmp_path / "ck"), "--checkpoint-every", "1"]
    r = subprocess.run(cmd, env=e, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    lines = [json.loads(x) for x in r.stdout.splitlines() if x.startswith("{")]
    assert [l["step"] for l in lines if "event" not in l] == [0, 1, 2]
    events = [l for l in lines if "event" in l]
    assert [l["event"] for l in events] == ["leaving", "failure"]
    assert events[0] == {"event": "leaving", "rank": 1, "step": 1}
    assert events[1]["rank"] == 0 and events[1]["kind"] == "PeerFailure"      # reported on the host, no wait budget spent
    assert "exitcode  : 75" in r.stderr and "launch.sh: attempt 1 of 1" in r.stderr
    assert (tmp_path / "restart.done").exists()


def test_hugging_face_model_trainer_agrees_with_the_converted_decoder(tmp_path):
    """``train_hf.py`` (the reference's recipe: a ``transformers`` model class under ``fully_shard`` + the patch, the
    chunked log-probability head) and ``train_fsdp2.py --hf-checkpoint`` (the same weights converted to this package's
    decoder) see the same first-minibatch loss on the same packed data."""
    pytest.importorskip("transformers")
    import torch
    sys.path.insert(0, REPO)
    from odc_b200.models import DecoderLM, get_config
    from odc_b200.models.hf import save_hf_checkpoint
    cfg = get_config("tiny", qkv_bias=True, tie_embeddings=False, vocab_size=512)
    src = DecoderLM(cfg)
    src.reset_parameters(seed=3)
    ckpt = tmp_path / "ckpt"
    save_hf_checkpoint(str(ckpt), src.state_dict(), cfg, dtype=torch.float32)

    def first_loss(script, **env):
        e = dict(os.environ, ODC="1", ODC_SYMMETRIC_SIZE="256M", ODC_OUT_DIR=str(tmp_path), FUSED_OPTIMIZER="0", **env)
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
               "127.0.0.1", "--master-port", str(_free_port()), os.path.join(REPO, "examples/llm_training", script), "--cpu",
               "--hf-checkpoint", str(ckpt), "--steps", "2", "--minibatch_size", "4", "--num-sequences", "16",
               "--length-dist", "uniform", "--limit_dataset_token_len", "200", "--max_token_len", "512",
               "--run_name", "hf_ab"]
        r = subprocess.run(cmd, env=e, capture_output=True, text=True, timeout=600)
        assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
        return [json.loads(x)["loss"] for x in r.stdout.splitlines() if x.startswith("{")]

    hf_losses = first_loss("train_hf.py")
    own_losses = first_loss("train_fsdp2.py")
    # both compute in bf16 (fp32 master weights), in different operation orders
    assert len(hf_losses) == 2 and hf_losses[0] == pytest.approx(own_losses[0], rel=5e-3)
    assert hf_losses[1] == pytest.approx(own_losses[1], rel=2e-2)   # after one AdamW step of each
    flat_losses = first_loss("train_hf.py", FSDP1="1")                 # the same model under FSDP1 flat parameters
    assert flat_losses[0] == pytest.approx(hf_losses[0], rel=5e-3) and flat_losses[1] == pytest.approx(hf_losses[1], rel=2e-2)
