"""Static documentation site: renders the Markdown pages of ``docs/`` into linked HTML pages.

    python -m nexus_b200.tools.site build [docs] [-o site]
    python -m nexus_b200.tools.site serve [site] [--port 8000]

The renderer covers what the pages use: ATX headings, paragraphs, fenced code, bullet and numbered lists,
pipe tables, block quotes, inline code / emphasis / links.  No third-party dependency.  Counterpart of the
Next.js documentation site under ``web/`` of the reference (pages under ``docs/architecture``).
"""
from __future__ import annotations

import argparse
import html
import re
import sys
from pathlib import Path
from typing import List, Tuple

_CSS = """
body{margin:0;font:16px/1.55 system-ui,sans-serif;color:#1b1f24;display:flex;min-height:100vh}
nav{width:250px;background:#0f1720;color:#d7dde4;padding:24px 18px;box-sizing:border-box;flex-shrink:0}
nav h1{font-size:18px;margin:0 0 16px}nav a{display:block;color:#d7dde4;text-decoration:none;padding:4px 0}
nav a.cur{color:#7cc4ff;font-weight:600}main{max-width:920px;padding:32px 48px;box-sizing:border-box}
pre{background:#f3f5f7;padding:12px 14px;overflow:auto;border-radius:6px;font-size:14px}
code{background:#f3f5f7;padding:1px 4px;border-radius:4px;font-size:90%}pre code{padding:0;background:none}
table{border-collapse:collapse;margin:12px 0}th,td{border:1px solid #d0d7de;padding:5px 10px;text-align:left}
th{background:#f3f5f7}blockquote{border-left:4px solid #d0d7de;margin:12px 0;padding:2px 14px;color:#57606a}
h1,h2,h3{line-height:1.25}a{color:#0b6bcb}
"""


def _inline(text: str) -> str:
    out, pos = [], 0
    for m in re.finditer(r"`([^`]+)`", text):            # code spans are taken out first: nothing inside is markup
        out.append(_inline_plain(text[pos:m.start()]))
        out.append("<code>" + html.escape(m.group(1)) + "</code>")
        pos = m.end()
    out.append(_inline_plain(text[pos:]))
    return "".join(out)


def _inline_plain(text: str) -> str:
    t = html.escape(text, quote=False)
    t = re.sub(r"\[([^\]]+)\]\(([^)\s]+)\)", lambda m: f'<a href="{_href(m.group(2))}">{m.group(1)}</a>', t)
    t = re.sub(r"\*\*([^*]+)\*\*", r"<strong>\1</strong>", t)
    t = re.sub(r"(?<![\w*])\*([^*\s][^*]*)\*(?![\w*])", r"<em>\1</em>", t)
    return t


def _href(target: str) -> str:
    if re.match(r"^[a-z]+://", target) or target.startswith("#"):
        return target
    path, _, frag = target.partition("#")
    if path.endswith(".md"):
        path = path[:-3] + ".html"
    return path + ("#" + frag if frag else "")


def _slug(text: str) -> str:
    return re.sub(r"[^a-z0-9]+", "-", text.lower()).strip("-")


def render_markdown(src: str) -> Tuple[str, str]:
    """Returns (html body, title).  The title is the first level-1 heading (or empty)."""
    lines = src.replace("\r\n", "\n").split("\n")
    out: List[str] = []
    title = ""
    i, n = 0, len(lines)

    def flush_paragraph(buf: List[str]) -> None:
        if buf:
            out.append("<p>" + _inline(" ".join(s.strip() for s in buf)) + "</p>")
            buf.clear()

    para: List[str] = []
    while i < n:
        line = lines[i]
        if line.startswith("```"):
            flush_paragraph(para)
            lang = line[3:].strip()
            i += 1
            code = []
            while i < n and not lines[i].startswith("```"):
                code.append(lines[i])
                i += 1
            i += 1
            cls = f' class="language-{html.escape(lang)}"' if lang else ""
            out.append(f"<pre><code{cls}>" + html.escape("\n".join(code)) + "</code></pre>")
            continue
        m = re.match(r"^(#{1,6})\s+(.*?)\s*#*$", line)
        if m:
            flush_paragraph(para)
            level, text = len(m.group(1)), m.group(2)
            if level == 1 and not title:
                title = text
            out.append(f'<h{level} id="{_slug(text)}">{_inline(text)}</h{level}>')
            i += 1
            continue
        if re.match(r"^\s*\|.*\|\s*$", line) and i + 1 < n and re.match(r"^\s*\|?\s*:?-{2,}", lines[i + 1]):
            flush_paragraph(para)
            header = [c.strip() for c in line.strip().strip("|").split("|")]
            i += 2
            rows = []
            while i < n and re.match(r"^\s*\|.*\|\s*$", lines[i]):
                rows.append([c.strip() for c in lines[i].strip().strip("|").split("|")])
                i += 1
            t = ["<table><thead><tr>" + "".join(f"<th>{_inline(c)}</th>" for c in header) + "</tr></thead><tbody>"]
            for r in rows:
                t.append("<tr>" + "".join(f"<td>{_inline(c)}</td>" for c in r) + "</tr>")
            t.append("</tbody></table>")
            out.append("".join(t))
            continue
        m = re.match(r"^(\s*)([-*]|\d+\.)\s+(.*)$", line)
        if m:
            flush_paragraph(para)
            ordered = m.group(2)[0].isdigit()
            items: List[str] = []
            while i < n:
                m2 = re.match(r"^(\s*)([-*]|\d+\.)\s+(.*)$", lines[i])
                if m2:
                    items.append(m2.group(3))
                elif lines[i].startswith("  ") and lines[i].strip() and items:
                    items[-1] += " " + lines[i].strip()      # continuation line of the item
                else:
                    break
                i += 1
            tag = "ol" if ordered else "ul"
            out.append(f"<{tag}>" + "".join(f"<li>{_inline(it)}</li>" for it in items) + f"</{tag}>")
            continue
        if line.startswith(">"):
            flush_paragraph(para)
            quote = []
            while i < n and lines[i].startswith(">"):
                quote.append(lines[i][1:].strip())
                i += 1
            out.append("<blockquote><p>" + _inline(" ".join(quote)) + "</p></blockquote>")
            continue
        if not line.strip():
            flush_paragraph(para)
        else:
            para.append(line)
        i += 1
    flush_paragraph(para)
    return "\n".join(out), title


def build(src_dir: Path, out_dir: Path) -> List[Path]:
    """Renders every ``*.md`` under `src_dir` (recursively) to `out_dir`; returns the written files."""
    pages = sorted(src_dir.rglob("*.md"), key=lambda p: (p.name != "index.md", str(p)))
    if not pages:
        raise FileNotFoundError(f"no Markdown pages under {src_dir}")
    rendered = []
    for p in pages:
        body, title = render_markdown(p.read_text(encoding="utf-8"))
        rendered.append((p.relative_to(src_dir).with_suffix(".html"), title or p.stem, body))
    written = []
    for rel, title, body in rendered:
        depth = len(rel.parts) - 1
        prefix = "../" * depth
        nav = "".join(f'<a href="{prefix}{r.as_posix()}"{" class=cur" if r == rel else ""}>{html.escape(t)}</a>'
                      for r, t, _ in rendered)
        page = (f"<!doctype html><html><head><meta charset=utf-8><title>{html.escape(title)} - nexus-b200</title>"
                f"<style>{_CSS}</style></head><body><nav><h1>nexus-b200</h1>{nav}</nav><main>{body}</main></body></html>")
        dst = out_dir / rel
        dst.parent.mkdir(parents=True, exist_ok=True)
        dst.write_text(page, encoding="utf-8")
        written.append(dst)
    return written


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="nexus_b200.tools.site")
    sub = ap.add_subparsers(dest="cmd", required=True)
    b = sub.add_parser("build")
    b.add_argument("src", nargs="?", default="docs")
    b.add_argument("-o", "--out", default="site")
    s = sub.add_parser("serve")
    s.add_argument("dir", nargs="?", default="site")
    s.add_argument("--port", type=int, default=8000)
    args = ap.parse_args(argv)
    if args.cmd == "build":
        files = build(Path(args.src), Path(args.out))
        print(f"{len(files)} pages -> {args.out}")
        return 0
    import functools
    import http.server
    handler = functools.partial(http.server.SimpleHTTPRequestHandler, directory=args.dir)
    with http.server.ThreadingHTTPServer(("127.0.0.1", args.port), handler) as srv:
        print(f"serving {args.dir} on http://127.0.0.1:{args.port}")
        srv.serve_forever()
    return 0


if __name__ == "__main__":
    sys.exit(main())
