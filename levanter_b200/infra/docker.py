"""Building, tagging and pushing the training image, and composing ``docker run`` lines for GPU hosts.

The reference's helper (src/levanter/infra/docker.py) builds an image from a Dockerfile, copies extra context into the build
directory, pushes to GitHub's or Google's registry and composes the ``docker run`` command its TPU launcher executes.  Here
the targets are hosts with NVIDIA GPUs: the run line asks for ``--gpus``, host IPC and unlimited locked memory (NCCL and the
peer-mapped buffers need both), and a registry is any ``host/namespace`` prefix.  Every function that would execute ``docker``
takes a ``run`` callable (default: ``subprocess.check_call`` with the command echoed), so launch scripts can dry-run."""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from typing import Callable, Dict, List, Optional, Sequence, Tuple

from .cli_helpers import format_command

Runner = Callable[[Sequence[str]], object]


def _default_run(cmd: Sequence[str]) -> None:
    print("+ " + format_command(list(cmd)), file=sys.stderr)
    subprocess.check_call(list(cmd))


def split_image_and_tag(image: str) -> Tuple[str, str]:
    """``registry:5000/ns/name:tag`` -> (``registry:5000/ns/name``, ``tag``); the tag defaults to ``latest``.  A colon that
    belongs to a registry port (followed by a slash later on) is not a tag separator."""
    head, sep, tail = image.rpartition(":")
    if sep and "/" not in tail:
        return head, tail
    return image, "latest"


class ExtraContext:
    """Copies a directory from outside the build context to ``<context>/.extra_context`` for the duration of a build (the
    Dockerfile can ``COPY .extra_context ...``) and removes it afterwards."""

    def __init__(self, source: Optional[str], context: str = "."):
        self.source, self.target = source, os.path.join(context, ".extra_context")

    def __enter__(self) -> Optional[str]:
        if self.source is None:
            return None
        if os.path.exists(self.target):
            shutil.rmtree(self.target)
        shutil.copytree(self.source, self.target)
        return self.target

    def __exit__(self, *exc) -> bool:
        if self.source is not None and os.path.exists(self.target):
            shutil.rmtree(self.target)
        return False


def build_docker(docker_file: str, image_name: str, tag: str = "latest", *, context: str = ".", build_args: Optional[Dict[str, str]] = None,
                 platform: str = "linux/amd64", extra_context: Optional[str] = None, run: Runner = _default_run) -> str:
    """``docker buildx build`` of ``docker_file``; returns ``image_name:tag``."""
    image = f"{image_name}:{tag}"
    cmd: List[str] = ["docker", "buildx", "build", "--platform", platform, "-f", docker_file, "-t", image]
    for k, v in (build_args or {}).items():
        cmd += ["--build-arg", f"{k}={v}"]
    with ExtraContext(extra_context, context):
        run(cmd + [context])
    return image


def push_to_registry(local_image: str, registry_prefix: str, *, run: Runner = _default_run) -> str:
    """Tag ``local_image`` as ``<registry_prefix>/<name>:<tag>`` and push it; returns the remote name."""
    name, tag = split_image_and_tag(local_image)
    remote = f"{registry_prefix.rstrip('/')}/{name.rsplit('/', 1)[-1]}:{tag}"
    run(["docker", "tag", local_image, remote])
    run(["docker", "push", remote])
    return remote


def push_to_github(local_image: str, github_user: str, github_token: Optional[str] = None, *, run: Runner = _default_run) -> str:
    """Push to ``ghcr.io/<user>``; with a token, log in first (the token goes to ``docker login`` on standard input)."""
    if github_token:
        print("+ docker login ghcr.io -u %s --password-stdin" % github_user, file=sys.stderr)
        if run is _default_run:
            subprocess.run(["docker", "login", "ghcr.io", "-u", github_user, "--password-stdin"], input=github_token.encode(), check=True)
        else:
            run(["docker", "login", "ghcr.io", "-u", github_user, "--password-stdin"])
    return push_to_registry(local_image, f"ghcr.io/{github_user}", run=run)


def make_docker_run_command(image: str, command: Sequence[str], *, foreground: bool = True, env: Optional[Dict[str, str]] = None,
                            name: str = "levanter", gpus: str = "all", mounts: Optional[Dict[str, str]] = None,
                            workdir: Optional[str] = None) -> List[str]:
    """The ``docker run`` line of one training process group on a GPU host: all (or the named) GPUs, host networking and
    IPC, no limit on locked memory, the environment passed through, optional bind mounts ``{host_path: container_path}``."""
    cmd = ["docker", "run", "-t" if foreground else "-d", f"--name={name}", "--gpus", gpus, "--net=host", "--ipc=host",
           "--ulimit", "memlock=-1", "--ulimit", "stack=67108864", "--shm-size=32g"]
    for host, cont in (mounts or {}).items():
        cmd += ["-v", f"{host}:{cont}"]
    if workdir:
        cmd += ["-w", workdir]
    for k, v in (env or {}).items():
        cmd += ["-e", f"{k}={v}"]
    return cmd + [image] + list(command)
