"""Interactive client of `examples/model_server.py`.

    python examples/chat.py --port 8765 [--tokenizer /path/to/hf_tokenizer_dir] [--gen-len 64]
    python examples/chat.py --port 8765 --once "hello"          # one request, print the reply, exit

Every turn is one connection: the client sends ``{"input_ids": [[...]], "gen_len": n}`` as a JSON line and reads one JSON
line back (the server's protocol).  The conversation so far (prompts and replies) is sent with every turn, so the model
sees the whole dialogue; ``/reset`` forgets it, ``/stop`` ends the server, ``/quit`` leaves.  Text is turned into token
ids by a Hugging Face tokenizer loaded from a local directory (``--tokenizer``; nothing is downloaded) or, without one,
by a byte-level stand-in (UTF-8 bytes, offset so that ids stay below ``--vocab``), which is enough to drive a
random-weight model.  Counterpart of the reference's demo client
(python/triton_dist/mega_triton_kernel/test/models/chat.py: socket client with a prompt loop).
"""
import argparse
import json
import socket
import sys
from typing import List, Optional


class ByteTokenizer:
    """UTF-8 bytes as token ids (shifted by ``offset``); ids outside the byte range decode to U+FFFD."""

    def __init__(self, vocab: int = 256, offset: int = 0):
        if vocab < 256 + offset:
            offset = max(0, vocab - 256)
        self.vocab, self.offset = vocab, offset

    def encode(self, text: str) -> List[int]:
        return [min(self.vocab - 1, b + self.offset) for b in text.encode("utf-8")]

    def decode(self, ids: List[int]) -> str:
        raw = bytearray()
        out = []
        for i in ids:
            b = i - self.offset
            if 0 <= b < 256:
                raw.append(b)
            else:
                out.append(raw.decode("utf-8", errors="replace"))
                raw = bytearray()
                out.append("�")
        out.append(raw.decode("utf-8", errors="replace"))
        return "".join(out)


class HFTokenizer:
    def __init__(self, path: str):
        from transformers import AutoTokenizer

        self.tok = AutoTokenizer.from_pretrained(path, local_files_only=True)

    def encode(self, text: str) -> List[int]:
        return list(self.tok.encode(text))

    def decode(self, ids: List[int]) -> str:
        return self.tok.decode(ids, skip_special_tokens=True)


class ChatClient:
    def __init__(self, host: str = "127.0.0.1", port: int = 8765, timeout: float = 300.0, tokenizer=None,
                 gen_len: int = 64, max_context: int = 0):
        self.host, self.port, self.timeout = host, port, timeout
        self.tok = tokenizer if tokenizer is not None else ByteTokenizer()
        self.gen_len = gen_len
        self.max_context = max_context          # keep at most this many history tokens (0 = all)
        self.history: List[int] = []

    # ------------------------------------------------------------------ transport
    def request(self, payload: dict) -> dict:
        """One JSON line out, one JSON line back; errors come back as ``{"error": ...}`` instead of exceptions."""
        try:
            with socket.create_connection((self.host, self.port), timeout=self.timeout) as s:
                s.sendall((json.dumps(payload) + "\n").encode("utf-8"))
                buf = b""
                while not buf.endswith(b"\n"):
                    chunk = s.recv(65536)
                    if not chunk:
                        break
                    buf += chunk
        except (OSError, socket.timeout) as e:
            return {"error": f"connection to {self.host}:{self.port} failed: {e}"}
        try:
            return json.loads(buf.decode("utf-8"))
        except json.JSONDecodeError as e:
            return {"error": f"malformed reply: {e}"}

    # ------------------------------------------------------------------ conversation
    def reset(self):
        self.history = []

    def say(self, text: str) -> dict:
        """Send the dialogue so far plus ``text``; returns ``{"text", "ids", "ms_per_token"}`` or ``{"error"}``."""
        ids = self.history + self.tok.encode(text)
        if self.max_context and len(ids) > self.max_context:
            ids = ids[-self.max_context:]
        if not ids:
            return {"error": "empty prompt"}
        rep = self.request({"input_ids": [ids], "gen_len": self.gen_len})
        if "error" in rep:
            return rep
        out = rep.get("output_ids")
        if not isinstance(out, list) or not out or not isinstance(out[0], list):
            return {"error": f"unexpected reply: {rep}"}
        new = [int(t) for t in out[0]]
        if len(new) >= len(ids) and new[:len(ids)] == ids:      # a server that echoes the prompt
            new = new[len(ids):]
        self.history = ids + new
        return {"text": self.tok.decode(new), "ids": new, "ms_per_token": rep.get("ms_per_token")}

    def stop_server(self) -> dict:
        return self.request({"cmd": "stop"})


def repl(client: ChatClient, inp=input, out=print) -> None:
    out("commands: /reset  /stop (ends the server)  /quit")
    while True:
        try:
            line = inp("you> ").strip()
        except (EOFError, KeyboardInterrupt):
            out("")
            return
        if not line:
            continue
        if line == "/quit":
            return
        if line == "/reset":
            client.reset()
            out("(history cleared)")
            continue
        if line == "/stop":
            out(json.dumps(client.stop_server()))
            return
        rep = client.say(line)
        if "error" in rep:
            out(f"error: {rep['error']}")
            continue
        ms = rep.get("ms_per_token")
        out(f"model> {rep['text']}" + (f"    [{ms:.2f} ms/token]" if isinstance(ms, (int, float)) else ""))


def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=8765)
    ap.add_argument("--timeout", type=float, default=300.0)
    ap.add_argument("--gen-len", type=int, default=64)
    ap.add_argument("--tokenizer", default=None, help="local directory of a Hugging Face tokenizer")
    ap.add_argument("--vocab", type=int, default=256, help="vocabulary size of the served model (byte tokenizer only)")
    ap.add_argument("--max-context", type=int, default=0, help="keep at most this many history tokens")
    ap.add_argument("--once", default=None, help="send this prompt, print the reply and exit")
    args = ap.parse_args(argv)
    tok = HFTokenizer(args.tokenizer) if args.tokenizer else ByteTokenizer(args.vocab)
    client = ChatClient(args.host, args.port, args.timeout, tok, args.gen_len, args.max_context)
    if args.once is not None:
        rep = client.say(args.once)
        print(json.dumps(rep))
        return 1 if "error" in rep else 0
    repl(client)
    return 0


if __name__ == "__main__":
    sys.exit(main())
