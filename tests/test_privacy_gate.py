"""The privacy gate: user content never reaches a log.

Prompts, generated text, message bodies and raw token ids are the user's data; token ids count as
content because they decode back to the exact text.  A rule that is only written down comes back, so
this test scans every source file of the package: a call that writes to a log, a warning or the
process's output streams may not take an argument that names such data (the reference keeps the
same gate beside its logger: `src/privacy.rs:1-12`).  Counts, lengths and ids of requests are fine.
"""
import ast
import os

ROOT = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "loken_b200")

# names that hold user content wherever they appear in this code base
CONTENT = {"prompt", "prompts", "text", "texts", "content", "messages", "message", "tokens", "token_ids",
           "prompt_ids", "ids", "output", "outputs", "completion", "delta", "input_ids", "generated", "reply",
           "prompt_embeds", "embeds", "caption", "suffix", "system", "body"}
# attribute reads that are NOT content although the base name is (a count, a size, an id)
HARMLESS_ATTRS = {"shape", "dtype", "device", "seq_id", "model_id", "status_code"}
LOGGERS = {"log", "logger", "logging", "LOG", "_log", "warnings"}
LOG_METHODS = {"debug", "info", "warning", "warn", "error", "exception", "critical", "log"}


def _is_log_call(node: ast.Call) -> bool:
    f = node.func
    if isinstance(f, ast.Name) and f.id == "print":
        return True
    if isinstance(f, ast.Attribute) and f.attr in LOG_METHODS:
        base = f.value
        while isinstance(base, ast.Attribute):
            base = base.value
        return isinstance(base, ast.Name) and base.id in LOGGERS
    if isinstance(f, ast.Attribute) and f.attr == "write":
        base = f.value
        return isinstance(base, ast.Attribute) and base.attr in ("stderr", "stdout")
    return False


def _content_names(node: ast.AST):
    """Names of user content that the expression reads as a value (len(x), x.shape and the like do not)."""
    if isinstance(node, ast.Call):
        fn = node.func
        if isinstance(fn, ast.Name) and fn.id in ("len", "type", "id", "bool"):
            return
        for a in list(node.args) + [k.value for k in node.keywords]:
            yield from _content_names(a)
        if isinstance(fn, ast.Attribute):
            yield from _content_names(fn.value)
        return
    if isinstance(node, ast.Attribute):
        if node.attr in HARMLESS_ATTRS:
            return
        if node.attr in CONTENT:
            yield node.attr
        yield from _content_names(node.value)
        return
    if isinstance(node, ast.Name):
        if node.id in CONTENT:
            yield node.id
        return
    for child in ast.iter_child_nodes(node):
        yield from _content_names(child)


def scan_source(src: str, path: str = "<src>"):
    hits = []
    for node in ast.walk(ast.parse(src, path)):
        if isinstance(node, ast.Call) and _is_log_call(node):
            for a in list(node.args) + [k.value for k in node.keywords if k.arg != "file"]:
                for name in _content_names(a):
                    hits.append((path, node.lineno, name))
    return hits


def test_no_log_line_carries_user_content():
    hits = []
    for d, _, files in os.walk(ROOT):
        for f in files:
            if f.endswith(".py"):
                p = os.path.join(d, f)
                with open(p, encoding="utf-8") as fh:
                    hits += scan_source(fh.read(), os.path.relpath(p, ROOT))
    assert not hits, "user content reaches a log or an output stream:\n" + "\n".join(
        f"  {p}:{ln}: `{name}`" for p, ln, name in hits)


def test_the_gate_sees_what_it_should():
    bad = [
        'log.info("got %s", prompt)', 'logger.debug(f"ids {token_ids}")', 'print(req.messages)',
        'logging.warning("reply: " + reply)', 'sys.stderr.write(str(seq.tokens))', 'print("x", file=sys.stderr, end=text)',
    ]
    good = [
        'log.info("prompt of %d tokens", len(prompt))', 'print(f"{len(tokens)} tokens in {dt:.1f} s")',
        'logger.info("request %s done", seq.seq_id)', 'print(x.shape)', 'out.write(text)',
    ]
    for src in bad:
        assert scan_source("import sys\n" + src), src
    for src in good:
        assert not scan_source(src), src
