"""Engine under real process groups: gloo on CPU (always) and NCCL + NVLink peer kernels on >= 2 GPUs."""
import os
import subprocess
import sys

import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def _run(nproc, *args, timeout=600):
    port = 29500 + (os.getpid() % 500)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(HERE, "dist_fsdp_check.py"), *args]
    env = dict(os.environ, OMP_NUM_THREADS="2")
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=env)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    return r.stdout


def test_gloo_world2_matches_single_process():
    out = _run(2, "--device", "cpu", "--steps", "2")
    assert "ok=True" in out


@pytest.mark.parametrize("layers", [0, 1])
def test_gloo_world2_graph_kept_for_some_layers(layers):
    """Layers that keep their autograd graph (no recompute) are reduced by their backward-done hooks."""
    out = _run(2, "--device", "cpu", "--steps", "2", "--recompute-layers", str(layers))
    assert "ok=True" in out


def test_gloo_world2_with_clipping():
    out = _run(2, "--device", "cpu", "--steps", "2", "--clip", "0.5")
    assert "ok=True" in out


def test_gloo_world4_hybrid_sharding_matches_single_process():
    """HSDP: shard groups of 2, 2 replicas; reduce-scatter inside the shard group, all-reduce of the shard across
    replicas, one update; with clipping the norm is taken after both reductions."""
    out = _run(4, "--device", "cpu", "--steps", "2", "--shard-size", "2", "--clip", "0.5")
    assert "ok=True" in out and "shard=2 replicas=2" in out


def test_gloo_world2_optimizer_state_on_host_and_units_kept_gathered():
    out = _run(2, "--device", "cpu", "--steps", "2", "--offload", "--keep-gathered")
    assert "ok=True" in out


@pytest.mark.gpu
def test_gpu_world2_hybrid_options():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    out = _run(2, "--device", "cuda", "--comm", "p2p", "--steps", "3", "--offload", "--keep-gathered")
    assert "ok=True" in out


@pytest.mark.gpu
@pytest.mark.parametrize("comm", ["p2p", "nccl"])
def test_gpu_world2(comm):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    out = _run(2, "--device", "cuda", "--comm", comm, "--steps", "3")
    assert "ok=True" in out
    if comm == "p2p":
        assert "p2p=True" in out


def _run_script(nproc, script, *args, timeout=600):
    port = 29000 + (os.getpid() % 400) + nproc
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(HERE, script), *args]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=dict(os.environ, OMP_NUM_THREADS="1"))
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    return r.stdout


@pytest.mark.parametrize("world", [2, 4])
def test_context_parallel_attention_gloo(world):
    assert "ok=True" in _run_script(world, "dist_cp_check.py")


def test_expert_parallel_gloo():
    assert "ok=True" in _run_script(2, "dist_moe_check.py")


@pytest.mark.gpu
def test_fused_gemm_collectives_2gpu():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    assert "ok=True" in _run_script(2, "dist_fused_check.py")


def test_tp_pp_backend_gloo():
    assert "ok=True" in _run_script(4, "dist_mcore_check.py")


def test_tp_backend_with_vision_tower_data_parallel_gloo():
    """--hetero-parallel: each tensor-parallel rank encodes a share of the images; losses over two steps (the second one
    sees the summed vision gradients) equal the single-process run."""
    out = _run_script(2, "dist_mcore_check.py", "--hetero")
    assert "hetero=True" in out and "ok=True" in out


@pytest.mark.parametrize("wide", [False, True])
def test_u_shaped_disaggregated_pipeline_gloo(wide):
    assert "ok=True" in _run_script(3, "dist_ldt_check.py", *(["--wide"] if wide else []))


def test_hybrid_usp_and_fpdt_attention_gloo():
    assert "ok=True" in _run_script(4, "dist_usp_check.py")


def test_wan_fsdp_ulysses_matches_single_process_gloo():
    assert "ok=True" in _run_script(2, "dist_wan_check.py")


@pytest.mark.gpu
def test_tensor_parallel_linears_use_fused_kernels_2gpu():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    assert "ok=True" in _run_script(2, "dist_tp_check.py")


@pytest.mark.gpu
def test_wan_fused_ulysses_matches_all_to_all_path_2gpu():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    assert "ok=True" in _run_script(2, "dist_wan_check.py", "--cuda")


@pytest.mark.gpu
def test_moe_peer_memory_dispatcher_matches_alltoall():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    assert "ok=True" in _run_script(2, "dist_moe_p2p_check.py")


@pytest.mark.parametrize("extra", [("--optimizer", "muon"), ("--optimizer", "muon", "--offload"), ("--lr-scaling",)])
def test_engine_optimizers_sharded_match_single_process_gloo(extra):
    """Muon (all-gathered update, round-robin Newton-Schulz, reduce-scattered result) and per-group learning-rate
    multipliers give the same parameters on two ranks as on one."""
    assert "ok=True" in _run_script(2, "dist_fsdp_check.py", *extra)


def test_encoder_data_balance_inside_the_model_gloo():
    """Images re-dealt across data-parallel ranks before the vision tower: same loss and gradients as without."""
    assert "ok=True" in _run_script(2, "dist_balance_check.py")


@pytest.mark.parametrize("world", [2, 4])
def test_gloo_packed_sequence_context_parallel(world):
    """Packed (document-boundary) stream cut into equal chunks, keys / values all-gathered, one varlen call per rank with
    bottom-right causal segments: outputs and q / k / v gradients equal the single-process attention."""
    assert "ok=True" in _run_script(world, "dist_packed_cp_check.py")


def test_gloo_world4_dynamic_dp_cp_switches_groups_and_exchanges_batches():
    """Per-iteration dp x cp choice from the longest sequence of all ranks; groups of every split prepared once; the
    members of a context-parallel group end up with the same list of batches."""
    assert "ok=True" in _run_script(4, "dist_dpcp_check.py")


def test_native_trainer_moe_recipe_with_expert_parallel_gloo():
    """examples/qwen3vl/tiny_moe_native.yaml end to end: dense engine + expert engine (EngineMux), EP = 2."""
    root = os.path.dirname(HERE)
    port = 29300 + (os.getpid() % 300)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(port), "-m", "mindspeed_mm_b200.runtime.trainer",
           os.path.join(root, "examples", "qwen3vl", "tiny_moe_native.yaml")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, cwd=root, env=dict(os.environ, OMP_NUM_THREADS="1"))
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "iteration        3/       3" in r.stdout + r.stderr


@pytest.mark.gpu
def test_ring_attention_over_peer_memory_2gpu():
    """Ring attention with K/V blocks pulled over NVLink peer memory and tcgen05 block kernels (forward + backward)."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    assert "ok=True" in _run_script(2, "dist_cp_check.py", "--cuda")


@pytest.mark.parametrize("mode", ["heartbeat", "timeout"])
def test_rank_leaving_between_steps_is_detected_on_the_host(mode):
    """Fault injection on the host under gloo: the survivor stops through the heartbeat store, or its next
    collective fails after the short process-group timeout."""
    port = 29100 + (os.getpid() % 300)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(port), os.path.join(HERE, "dist_failure_check.py"), mode]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=180, env=dict(os.environ, OMP_NUM_THREADS="1"))
    assert f"detected={mode} ok=True" in r.stdout + r.stderr, r.stdout[-2000:] + r.stderr[-2000:]


def test_model_families_sharded_step_matches_single_process_gloo():
    """Speech LMs, LTX-2, Bagel, reward model, CogVideoX-style DiT, VACE, Wan2.2 with routed experts under ZeRO-3 at world 2."""
    assert "ok=True" in _run_script(2, "dist_zoo_check.py")
