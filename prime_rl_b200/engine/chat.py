"""Terminal chat against a running inference server (OpenAI-style ``/v1/chat/completions``),
for a quick look at what a checkpoint or a freshly broadcast policy says
(reference: scripts/chat.py).

    python -m prime_rl_b200.engine.chat --base-url http://127.0.0.1:8000 --system "You are terse."

Commands inside the session: ``/reset`` clears the conversation, ``/system <text>`` replaces the
system prompt, ``/temp <x>`` and ``/max <n>`` change sampling, ``/quit`` leaves.
"""

from __future__ import annotations

import argparse
import sys

import httpx


class ChatSession:
    def __init__(self, base_url: str, model: str | None = None, system: str | None = None, temperature: float = 0.7,
                 max_tokens: int = 512, transport=None, timeout: float = 600.0):
        self.client = httpx.Client(base_url=base_url.rstrip("/"), timeout=timeout, transport=transport)
        self.model, self.system, self.temperature, self.max_tokens = model, system, temperature, max_tokens
        self.messages: list[dict] = []

    def reset(self) -> None:
        self.messages = []

    def _model(self) -> str:
        if self.model is None:
            data = self.client.get("/v1/models").json().get("data") or [{}]
            self.model = data[0].get("id", "default")
        return self.model

    def command(self, line: str) -> str | None:
        """Handles a ``/command``; returns the text to print, or None when ``line`` is not one."""
        if not line.startswith("/"):
            return None
        name, _, arg = line[1:].partition(" ")
        if name == "reset":
            self.reset()
            return "conversation cleared"
        if name == "system":
            self.system = arg.strip() or None
            self.reset()
            return "system prompt set"
        if name == "temp":
            self.temperature = float(arg)
            return f"temperature {self.temperature}"
        if name == "max":
            self.max_tokens = int(arg)
            return f"max tokens {self.max_tokens}"
        if name in ("quit", "exit"):
            raise EOFError
        return f"unknown command /{name}"

    def say(self, text: str) -> str:
        self.messages.append({"role": "user", "content": text})
        msgs = ([{"role": "system", "content": self.system}] if self.system else []) + self.messages
        r = self.client.post("/v1/chat/completions", json={"model": self._model(), "messages": msgs,
                                                            "temperature": self.temperature,
                                                            "max_tokens": self.max_tokens})
        r.raise_for_status()
        reply = r.json()["choices"][0]["message"]["content"]
        self.messages.append({"role": "assistant", "content": reply})
        return reply


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--base-url", default="http://127.0.0.1:8000")
    ap.add_argument("--model", default=None)
    ap.add_argument("--system", default=None)
    ap.add_argument("--temperature", type=float, default=0.7)
    ap.add_argument("--max-tokens", type=int, default=512)
    args = ap.parse_args(argv)
    chat = ChatSession(args.base_url, args.model, args.system, args.temperature, args.max_tokens)
    print("connected to", args.base_url, "- /quit to leave")
    while True:
        try:
            line = input("> ").strip()
            if not line:
                continue
            out = chat.command(line)
            print(out if out is not None else chat.say(line))
        except (EOFError, KeyboardInterrupt):
            print()
            return 0
        except httpx.HTTPError as e:
            print(f"[request failed: {e}]")


if __name__ == "__main__":
    sys.exit(main())
