"""Language-server proxy that explains shape errors inline.

Counterpart of crates/incin-lsp (src/frame.rs: ``Content-Length`` framing; src/rewrite.rs: rewriting of the server's
diagnostics and hovers, with the request ids of pending hovers remembered so that only their answers are touched;
src/main.rs: two pumps between the editor and the wrapped server) and of the ``editors/`` glue.  The reference rewrites
rust-analyzer's type-level shape errors; shapes are run-time values here, so the proxy fronts any Python language
server and appends the :mod:`incin_b200.diagnostics` explanation to

* every ``textDocument/publishDiagnostics`` entry whose message is a recognised shape error (test runners and
  notebook servers publish exception texts as diagnostics), and
* hover answers whose text contains one (a hover over a failing cell or a traceback).

Editor glue is the editor's "language server command" setting:

    VS Code (settings.json)    "python.languageServer": "None", and a generic LSP client pointing at
                               ["python", "-m", "incin_b200", "lsp", "--", "pylsp"]
    Neovim (lspconfig)         cmd = { "python", "-m", "incin_b200", "lsp", "--", "pylsp" }

``INCIN_LSP_SERVER`` names the wrapped server when no command follows ``--``; ``INCIN_LSP_HINTS=0`` passes everything
through untouched.
"""
from __future__ import annotations

import json
import os
import subprocess
import sys
import threading

from .diagnostics import RULES, explain

MAX_FRAME = 64 << 20     # a header that announces more than this is treated as a broken stream


def read_frame(stream) -> bytes | None:
    """One message body, or None at end of stream.  Header names are case-insensitive; unknown headers are skipped."""
    length = None
    while True:
        line = stream.readline()
        if not line:
            return None
        line = line.strip()
        if not line:
            if length is None:
                continue          # stray blank line between frames
            break
        name, _, value = line.partition(b":")
        if name.strip().lower() == b"content-length":
            try:
                length = int(value.strip())
            except ValueError:
                raise ValueError(f"bad Content-Length header: {line!r}") from None
    if length < 0 or length > MAX_FRAME:
        raise ValueError(f"frame of {length} bytes refused")
    body = stream.read(length)
    return body if len(body) == length else None


def write_frame(stream, body: bytes) -> None:
    stream.write(b"Content-Length: " + str(len(body)).encode() + b"\r\n\r\n" + body)
    stream.flush()


def _explained(text: str) -> str | None:
    d = explain(text)
    if d is None or "hint: " + d.hint in text:      # already rewritten (a server that echoes our text back)
        return None
    out = f"{text.rstrip()}\n{d}"
    if d.op in RULES:
        out += f"\n  rule: {RULES[d.op]}"
    return out


class PendingRequests:
    """Ids of the editor's hover requests that the server has not answered yet."""

    def __init__(self):
        self._lock = threading.Lock()
        self._hover: set = set()

    def observe_outgoing(self, msg: dict) -> None:
        if msg.get("method") == "textDocument/hover" and "id" in msg:
            with self._lock:
                self._hover.add(_hashable(msg["id"]))

    def take_hover(self, msg_id) -> bool:
        with self._lock:
            key = _hashable(msg_id)
            if key in self._hover:
                self._hover.discard(key)
                return True
            return False


def _hashable(v):
    return v if isinstance(v, (int, str)) else json.dumps(v, sort_keys=True)


def _rewrite_hover_contents(c):
    """MarkupContent, a MarkedString or a list of them: returns (new value, changed)."""
    if isinstance(c, str):
        new = _explained(c)
        return (new, True) if new else (c, False)
    if isinstance(c, dict) and isinstance(c.get("value"), str):
        new = _explained(c["value"])
        return (dict(c, value=new), True) if new else (c, False)
    if isinstance(c, list):
        out, changed = [], False
        for item in c:
            item, ch = _rewrite_hover_contents(item)
            out.append(item)
            changed |= ch
        return out, changed
    return c, False


def rewrite_from_server(msg: dict, pending: PendingRequests, hints: bool = True) -> dict | None:
    """The message to forward instead of ``msg``, or None when it passes through unchanged."""
    if not hints or not isinstance(msg, dict):
        return None
    if msg.get("method") == "textDocument/publishDiagnostics":
        diags = (msg.get("params") or {}).get("diagnostics")
        if not isinstance(diags, list):
            return None
        changed, out = False, []
        for d in diags:
            new = _explained(d["message"]) if isinstance(d, dict) and isinstance(d.get("message"), str) else None
            out.append(dict(d, message=new) if new else d)
            changed |= new is not None
        return dict(msg, params=dict(msg["params"], diagnostics=out)) if changed else None
    if "id" in msg and "method" not in msg and pending.take_hover(msg["id"]):
        result = msg.get("result")
        if isinstance(result, dict) and "contents" in result:
            contents, changed = _rewrite_hover_contents(result["contents"])
            if changed:
                return dict(msg, result=dict(result, contents=contents))
    return None


def pump_editor_to_server(editor_in, server_in, pending: PendingRequests) -> None:
    while (body := read_frame(editor_in)) is not None:
        try:
            pending.observe_outgoing(json.loads(body))
        except (ValueError, AttributeError):
            pass                       # not JSON: forwarded as it is
        write_frame(server_in, body)


def pump_server_to_editor(server_out, editor_out, pending: PendingRequests, hints: bool = True) -> None:
    while (body := read_frame(server_out)) is not None:
        new = None
        try:
            new = rewrite_from_server(json.loads(body), pending, hints)
        except ValueError:
            pass
        write_frame(editor_out, json.dumps(new, separators=(",", ":")).encode() if new is not None else body)


def main(argv: list[str]) -> int:
    cmd = argv[argv.index("--") + 1:] if "--" in argv else []
    if not cmd and os.environ.get("INCIN_LSP_SERVER"):
        cmd = os.environ["INCIN_LSP_SERVER"].split()
    if not cmd:
        print("usage: python -m incin_b200 lsp -- <language server command> (or INCIN_LSP_SERVER)", file=sys.stderr)
        return 2
    hints = os.environ.get("INCIN_LSP_HINTS", "1") != "0"
    try:
        child = subprocess.Popen(cmd, stdin=subprocess.PIPE, stdout=subprocess.PIPE)
    except OSError as e:
        print(f"incin lsp: failed to start {cmd[0]!r}: {e}", file=sys.stderr)
        return 1
    pending = PendingRequests()

    def up():
        try:
            pump_editor_to_server(sys.stdin.buffer, child.stdin, pending)
        except (OSError, ValueError):
            pass
        finally:
            try:
                child.stdin.close()
            except OSError:
                pass

    t = threading.Thread(target=up, daemon=True)
    t.start()
    try:
        pump_server_to_editor(child.stdout, sys.stdout.buffer, pending, hints)
    except (OSError, ValueError):
        pass
    return child.wait()
