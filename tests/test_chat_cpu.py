"""The demo chat client: tokenizer round trip, the prompt loop against an in-process fake server, and one real turn
against `examples/model_server.py` serving the tiny model on CPU."""
import importlib.util
import json
import os
import socket
import subprocess
import sys
import threading
import time

ROOT = os.path.join(os.path.dirname(__file__), "..")


def _load(name):
    spec = importlib.util.spec_from_file_location(name, os.path.join(ROOT, "examples", f"{name}.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_byte_tokenizer_round_trip():
    chat = _load("chat")
    tok = chat.ByteTokenizer(vocab=256)
    text = "héllo, wörld ✓"
    assert tok.decode(tok.encode(text)) == text
    shifted = chat.ByteTokenizer(vocab=1024, offset=3)
    assert shifted.decode(shifted.encode(text)) == text
    assert shifted.decode([0, 1]) == "��"          # ids below the offset are not bytes
    assert max(chat.ByteTokenizer(vocab=300, offset=100).encode("\xff")) < 300


def test_prompt_loop_against_fake_server():
    chat = _load("chat")
    port = _free_port()
    seen = []
    srv = socket.socket()
    srv.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
    srv.bind(("127.0.0.1", port))
    srv.listen(4)

    def serve():
        while True:
            conn, _ = srv.accept()
            req = json.loads(conn.makefile("r").readline())
            seen.append(req)
            if req.get("cmd") == "stop":
                conn.sendall(b'{"ok": true, "cmd": "stop"}\n')
                conn.close()
                return
            ids = req["input_ids"][0]
            if ids[-1] == ord("!"):
                conn.sendall(b'{"error": "prompt + gen_len exceeds max_length"}\n')
            else:
                conn.sendall((json.dumps({"output_ids": [[ids[-1]] * req["gen_len"]], "ms_per_token": 1.5}) + "\n").encode())
            conn.close()

    t = threading.Thread(target=serve, daemon=True)
    t.start()
    client = chat.ChatClient(port=port, gen_len=3, timeout=10)
    lines = iter(["ab", "", "c", "no!", "/reset", "d", "/stop"])
    printed = []
    chat.repl(client, inp=lambda _: next(lines), out=printed.append)
    t.join(timeout=10)
    srv.close()
    prompts = [r["input_ids"][0] for r in seen if "input_ids" in r]
    assert prompts[0] == [97, 98]
    assert prompts[1] == [97, 98, 98, 98, 98, 99]                      # history: prompt, three reply tokens, new text
    assert prompts[3] == [100]                                         # after /reset
    assert seen[-1] == {"cmd": "stop"}
    assert any(p.startswith("model> bbb") and "ms/token" in p for p in printed)
    assert any(p.startswith("error: prompt + gen_len") for p in printed)
    # an error leaves the history as it was before the failed turn
    assert prompts[2][:len(prompts[1]) + 3] == prompts[1] + [99, 99, 99]


def test_unreachable_server_is_an_error_reply():
    chat = _load("chat")
    rep = chat.ChatClient(port=_free_port(), timeout=2).say("x")
    assert "error" in rep and "failed" in rep["error"]


def test_one_turn_against_the_real_server():
    chat = _load("chat")
    port = _free_port()
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", CUDA_VISIBLE_DEVICES="")
    proc = subprocess.Popen([sys.executable, os.path.join(ROOT, "examples", "model_server.py"), "--model", "tiny-dense",
                             "--port", str(port), "--max-requests", "2", "--max-length", "128"],
                            stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, env=env)
    try:
        deadline = time.time() + 240
        line = ""
        while time.time() < deadline:
            line = proc.stdout.readline()
            if "serving" in line or not line:
                break
        assert "serving" in line, f"server did not come up: {line!r}"
        client = chat.ChatClient(port=port, gen_len=4, timeout=120)
        first = client.say("hi")
        assert "error" not in first, first
        assert len(first["ids"]) == 4 and all(0 <= t < 256 for t in first["ids"])
        second = client.say("again")
        assert "error" not in second, second
        assert len(client.history) == 2 + 4 + 5 + 4
        proc.wait(timeout=60)                                          # --max-requests 2: the server leaves by itself
        assert proc.returncode == 0
    finally:
        if proc.poll() is None:
            proc.kill()
