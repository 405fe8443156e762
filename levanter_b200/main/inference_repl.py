"""Interactive front end to the inference server: load/unload checkpoints, chat, batch files, serve HTTP
(src/levanter/main/inference_repl.py:56-470).  Runs as a prompt (no arguments) or executes one ``--command``."""
from __future__ import annotations

import asyncio
import json
import logging
import shlex
import threading
from dataclasses import dataclass, field
from typing import List, Optional

from levanter_b200 import config as lev_config
from levanter_b200.compat.hf_checkpoints import load_tokenizer
from levanter_b200.inference.engine import InferenceEngineConfig
from levanter_b200.inference.openai import (ChatCompletionRequest, ChatMessage, InferenceServer, InferenceServerConfig,
                                            _create_chat_completion)
from levanter_b200.main._common import load_model
from levanter_b200.models.llama import LlamaConfig
from levanter_b200.models.lm_model import LmConfig
from levanter_b200.parallel.mesh import local_device
from levanter_b200.trainer import TrainerConfig

logger = logging.getLogger(__name__)


@dataclass
class InferenceReplConfig:
    checkpoint: Optional[str] = None  # a checkpoint of this framework or a Hugging Face id/path
    model: Optional[LmConfig] = None
    tokenizer: Optional[str] = None
    trainer: TrainerConfig = field(default_factory=TrainerConfig)
    server: InferenceServerConfig = field(default_factory=lambda: InferenceServerConfig(
        model=LlamaConfig(), service=InferenceEngineConfig(max_pages=32, max_seqs=2, page_size=8, max_pages_per_seq=8, max_queued_tokens=4,
                                                           max_seqs_in_prefill=2, max_prefill_size=64, max_tokens_per_round=16, max_rounds=8)))
    temperature: float = 0.7
    seed: int = 42
    max_tokens: int = 64
    command: Optional[str] = None
    args: str = ""


class ReplContext:
    """Holds the server (created by the first ``load``) and implements the commands."""

    def __init__(self, config: InferenceReplConfig):
        self.config = config
        self.server: Optional[InferenceServer] = None
        self.model_name: Optional[str] = None
        self._http: Optional[threading.Thread] = None
        self.commands = {"load": self.load, "unload": self.unload, "chat": self.chat, "batch": self.batch, "serve": self.serve,
                         "help": self.show_help}

    def execute(self, cmd_name: str, *args, **kwargs):
        if cmd_name not in self.commands:
            print(f"Unknown command: {cmd_name}")
            return self.show_help()
        return self.commands[cmd_name](*args, **kwargs)

    def _is_hf(self, path: str) -> bool:
        import os

        return not (os.path.isdir(path) and not os.path.exists(os.path.join(path, "config.json")))

    def load(self, path: str, tokenizer: Optional[str] = None, **kwargs):
        """load <checkpoint or HF id> [tokenizer]: load weights, or swap them under a running server."""
        tok = load_tokenizer(tokenizer or self.config.tokenizer or path)
        model_config = self.config.model or self.config.server.model
        is_hf = self._is_hf(path)

        def build(_current=None):
            return load_model(model_config, tok, checkpoint_path=None if is_hf else path, hf_checkpoint=path if is_hf else None,
                              dtype=self.config.trainer.mp.compute_dtype, device=local_device()).eval()

        if self.server is None:
            self.server = InferenceServer.create(self.config.server, model=build(), tokenizer=tok)
        else:
            self.server.inference_context.tokenizer = tok
            self.server.reload(build)
        self.model_name = path
        print(f"Loaded {path}")

    def unload(self):
        if self.server is not None:
            self.server.unload()
        self.model_name = None
        print("Model unloaded")

    def serve(self):
        """serve: expose the OpenAI-compatible HTTP API in a background thread."""
        if self.server is None:
            return print("Load a model first")
        if self._http is None:
            self._http = threading.Thread(target=self.server.serve, daemon=True)
            self._http.start()
        print(f"Serving on http://{self.config.server.host}:{self.config.server.port}")

    def show_help(self):
        print("Commands:\n  load <path> [tokenizer]\n  unload\n  chat [message]   (no message: interactive session, empty line ends it)\n"
              "  batch <file.jsonl>  (one {\"messages\": [...]} or {\"prompt\": ...} per line)\n  serve\n  help\n  quit")

    def _run_chat_completion(self, messages: List[dict], print_response: bool = True):
        if self.server is None or self.model_name is None:
            return print("Load a model first")
        req = ChatCompletionRequest(model=self.model_name, messages=[ChatMessage(**m) for m in messages], max_tokens=self.config.max_tokens,
                                    temperature=self.config.temperature, seed=self.config.seed)
        resp = asyncio.run(_create_chat_completion(self.server.inference_context, req))
        if print_response:
            for c in resp["choices"]:
                print(c["message"]["content"])
            print(f"[{resp['usage']['completion_tokens']} tokens]")
        return resp

    def chat(self, message: Optional[str] = None):
        if message is not None:
            return self._run_chat_completion([{"role": "user", "content": message}])
        history: List[dict] = []
        while True:
            try:
                line = input("you> ").strip()
            except EOFError:
                break
            if not line:
                break
            history.append({"role": "user", "content": line})
            resp = self._run_chat_completion(history)
            if resp:
                history.append({"role": "assistant", "content": resp["choices"][0]["message"]["content"]})

    def batch(self, batch_input: str):
        out = []
        with open(batch_input) as f:
            for line in f:
                if not line.strip():
                    continue
                row = json.loads(line)
                messages = row.get("messages") or [{"role": "user", "content": row.get("prompt", "")}]
                resp = self._run_chat_completion(messages, print_response=False)
                out.append(resp)
                print(json.dumps({"input": row, "output": resp["choices"][0]["message"]["content"] if resp else None}))
        return out


def repl_mode(config: InferenceReplConfig, commands: ReplContext):
    commands.show_help()
    while True:
        try:
            line = input("levanter> ").strip()
        except EOFError:
            break
        if not line:
            continue
        if line in ("quit", "exit"):
            break
        parts = shlex.split(line)
        try:
            commands.execute(parts[0], *parts[1:])
        except Exception as e:  # noqa: BLE001 - a failed command must not end the session
            print(f"error: {e}")


def cli_mode(config: InferenceReplConfig, commands: ReplContext):
    if config.checkpoint is not None and config.command != "load":
        commands.load(config.checkpoint)
    commands.execute(config.command, *shlex.split(config.args))


def main(config: InferenceReplConfig):
    config.trainer.initialize()
    commands = ReplContext(config)
    if config.command is not None:
        cli_mode(config, commands)
    else:
        if config.checkpoint is not None:
            commands.load(config.checkpoint)
        repl_mode(config, commands)
    if commands.server is not None:
        commands.server.shutdown()


if __name__ == "__main__":
    lev_config.main(main)()
