"""The docker helpers compose the right command lines; nothing here runs docker."""
import os

from levanter_b200.infra import docker as D


def test_image_and_tag_are_split_at_the_tag_colon_only():
    assert D.split_image_and_tag("ghcr.io/me/levanter:abc") == ("ghcr.io/me/levanter", "abc")
    assert D.split_image_and_tag("registry:5000/ns/levanter") == ("registry:5000/ns/levanter", "latest")
    assert D.split_image_and_tag("levanter") == ("levanter", "latest")


def test_build_tags_pushes_and_cleans_the_extra_context(tmp_path):
    calls = []
    extra = tmp_path / "extra"
    extra.mkdir()
    (extra / "f.txt").write_text("x")
    ctx = tmp_path / "ctx"
    ctx.mkdir()
    seen = []

    def run(cmd):
        calls.append(list(cmd))
        seen.append(os.path.exists(ctx / ".extra_context" / "f.txt"))

    image = D.build_docker("docker/Dockerfile", "levanter", "t1", context=str(ctx), build_args={"CUDA": "12.9"}, extra_context=str(extra), run=run)
    assert image == "levanter:t1" and seen == [True] and not os.path.exists(ctx / ".extra_context")
    assert calls[0][:3] == ["docker", "buildx", "build"] and "--build-arg" in calls[0] and "CUDA=12.9" in calls[0] and calls[0][-1] == str(ctx)
    remote = D.push_to_registry(image, "registry:5000/team", run=run)
    assert remote == "registry:5000/team/levanter:t1"
    assert calls[1] == ["docker", "tag", "levanter:t1", remote] and calls[2] == ["docker", "push", remote]
    assert D.push_to_github(image, "me", run=run) == "ghcr.io/me/levanter:t1"


def test_run_line_asks_for_gpus_host_ipc_and_unlimited_locked_memory():
    cmd = D.make_docker_run_command("levanter:t1", ["python", "-m", "levanter_b200.main.train_lm"], foreground=False,
                                    env={"WANDB_API_KEY": "k"}, mounts={"/data": "/data"}, gpus="device=0,1")
    s = " ".join(cmd)
    assert "-d" in cmd and "--gpus device=0,1" in s and "--ipc=host" in cmd and "memlock=-1" in s and "-e WANDB_API_KEY=k" in s
    assert "-v /data:/data" in s and cmd[-3:] == ["python", "-m", "levanter_b200.main.train_lm"]
