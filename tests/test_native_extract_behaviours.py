"""Behaviour list of text extraction (C++ ``native.extract``; reference data/extract/tests/
{empty,extract_from,format,html,latex,pdf,preserves_math,roundtrip,unparseable,hash_helpers}.rs):
format detection from paths and media types, what survives from HTML, LaTeX math kept as
source, PDF text operators, content hashes of the extracted text and the error kinds."""
import hashlib
import zlib

import pytest

from prometheus_b200 import native
from prometheus_b200.native import NativeError

EX = native.extract


def err(call):
    with pytest.raises(NativeError) as e:
        call()
    return e.value


def pdf(content: bytes, flate=False) -> bytes:
    body = zlib.compress(content) if flate else content
    filt = b"/Filter /FlateDecode " if flate else b""
    return (b"%PDF-1.4\n1 0 obj\n<< /Type /Catalog >>\nendobj\n2 0 obj\n<< " + filt + b"/Length " + str(len(body)).encode()
            + b" >>\nstream\n" + body + b"\nendstream\nendobj\ntrailer\n<< /Root 1 0 R >>\n%%EOF\n")


HELLO_PDF = pdf(b"BT /F1 12 Tf 72 720 Td (Hello PDF) Tj ET")


# ------------------------------------------------------------------------------ format detection
@pytest.mark.parametrize("path, fmt", [("a.html", "html"), ("a.htm", "html"), ("a.xhtml", "html"), ("dir/Page.HTML", "html"),
                                       ("paper.pdf", "pdf"), ("P.PDF", "pdf"), ("src.tex", "latex"), ("x.latex", "latex"),
                                       ("archive.tar.html", "html"), ("page.html.bak", None), ("noext", None), ("x.md", None),
                                       ("", None), ("dir.html/file", None)])
def test_format_from_path_uses_the_final_extension(path, fmt):
    assert EX.format_from_path(path) == fmt


@pytest.mark.parametrize("media, fmt", [("text/html", "html"), ("application/xhtml+xml", "html"), ("text/html; charset=utf-8", None),
                                        ("application/pdf", "pdf"), ("application/x-latex", "latex"), ("text/x-tex", "latex"),
                                        ("application/x-tex", "latex"), ("image/png", None), ("text/plain", None), ("", None)])
def test_format_from_media_type(media, fmt):
    assert EX.format_from_media_type(media) == fmt                                      # exact names; parameters are not parsed


def test_extract_from_picks_the_format_and_records_the_source():
    html = b"<html><body><p>Hello there</p></body></html>"
    by_path = EX.extract_from(html, path="crawl/page.htm")
    by_type = EX.extract_from(html, media_type="application/xhtml+xml")
    both = EX.extract_from(html, path="crawl/page.html", media_type="text/html")
    direct = EX.extract(html, "html")
    assert by_path.text == by_type.text == both.text == direct.text and by_path.format == "html"
    assert by_path.source == "crawl/page.htm" and by_type.source is None and direct.source is None
    assert by_path.bytes_in == len(html)
    assert EX.extract_from(HELLO_PDF, path="a.pdf").format == "pdf" and EX.extract_from(HELLO_PDF, media_type="application/pdf").format == "pdf"
    assert EX.extract_from(b"$x$", path="a.tex").format == "latex" and EX.extract_from(b"$x$", media_type="text/x-tex").format == "latex"
    assert err(lambda: EX.extract_from(html)).kind == "Unsupported"
    assert err(lambda: EX.extract_from(html, path="notes.txt", media_type="text/plain")).kind == "Unsupported"


# ------------------------------------------------------------------------------ empty / unparseable
@pytest.mark.parametrize("fmt", ["html", "pdf", "latex"])
def test_empty_input_is_empty_for_every_format(fmt):
    assert err(lambda: EX.extract(b"", fmt)).kind == "Empty"
    path = {"html": "a.html", "pdf": "a.pdf", "latex": "a.tex"}[fmt]
    assert err(lambda: EX.extract_from(b"", path=path)).kind == "Empty"


def test_unparseable_inputs():
    assert err(lambda: EX.extract(b"\xff\xfe<p>x</p>", "html")).kind == "Unparseable"
    assert err(lambda: EX.extract(b"$x$ \xc3\x28", "latex")).kind == "Unparseable"
    assert err(lambda: EX.extract(b"this is not a pdf", "pdf")).kind == "Unparseable"
    assert err(lambda: EX.extract(HELLO_PDF[:40], "pdf")).kind == "Unparseable"                    # truncated
    assert err(lambda: EX.extract_from(b"garbage", path="x.pdf")).kind == "Unparseable"
    assert err(lambda: EX.extract_from(b"\xff\xfe", media_type="text/html")).kind == "Unparseable"
    assert err(lambda: EX.extract(b"<p>x</p>", "docx")).kind in ("Unsupported", "Config", "Other")


# ------------------------------------------------------------------------------ html
def test_html_keeps_text_and_drops_markup_scripts_styles_comments():
    page = (b"<html><head><title>T</title><style>p { color: red }</style><script>var hidden = 1;</script></head>"
            b"<body><!-- a comment --><h1>Title One</h1><p>First <b>bold <i>nested</i></b> text.</p>"
            b"<p>Fish &amp; chips &lt;3 &quot;quoted&quot; caf&eacute; &#8212; &#x2603;</p></body></html>")
    text = EX.extract(page, "html").text
    for want in ("Title One", "First bold nested text.", 'Fish & chips <3 "quoted"', "café", "—", "☃"):
        assert want in text
    for gone in ("color: red", "hidden", "a comment", "<b>", "</p>", "&amp;"):
        assert gone not in text
    assert text.index("Title One") < text.index("First bold")
    assert EX.extract("<p>naïve Ünïcode 日本語</p>".encode(), "html").text.strip() == "naïve Ünïcode 日本語"
    math = EX.extract(b"<p>Energy is $E = mc^2$ and \\(a_b\\).</p>", "html").text
    assert "$E = mc^2$" in math and EX.preserves_latex_math(math)
    assert EX.extract(b"<div><span></span></div>", "html").text.strip() == ""                       # markup only: not an Empty error


# ------------------------------------------------------------------------------ latex
def test_latex_math_survives_as_source():
    src = (rb"\documentclass{article}\begin{document}% a comment" b"\n" rb"Inline $\alpha + \beta$ and display \[ \int_0^1 x^2 dx \] then"
           rb"\begin{equation}E = mc^2\end{equation} and \begin{align*}a &= b\\c &= d\end{align*} done. 100\% sure.\end{document}")
    text = EX.extract(src, "latex").text
    for want in (r"$\alpha + \beta$", r"\int_0^1 x^2 dx", r"\begin{equation}E = mc^2\end{equation}", r"\begin{align*}", "100\\% sure."):
        assert want in text
    assert "a comment" not in text and "α" not in text and "∫" not in text                         # no unicode approximation
    assert EX.preserves_latex_math(text)
    assert EX.extract(rb"$x^2$", "latex").text.strip() == "$x^2$"


@pytest.mark.parametrize("text, yes", [("a $x$ b", True), ("$$ x $$", True), (r"\begin{equation}x\end{equation}", True),
                                       (r"\begin{align}x\end{align}", True), (r"\[ x \]", False), (r"\( x \)", False),
                                       ("plain text", False), ("", False), (r"\begin{document}hi\end{document}", False),
                                       (r"costs \$5 and \$6", False), ("one $ sign", False)])
def test_what_counts_as_preserved_math(text, yes):
    assert EX.preserves_latex_math(text) == yes


# ------------------------------------------------------------------------------ pdf
def test_pdf_text_operators():
    assert EX.extract(HELLO_PDF, "pdf").text.strip() == "Hello PDF"
    content = b"BT /F1 12 Tf 72 720 Td (Hello \\(nested\\)) Tj 0 -14 Td [(sec) -20 (ond)] TJ T* (third \\\\ line) ' ET"
    for flate in (False, True):
        text = EX.extract(pdf(content, flate), "pdf").text
        assert "Hello (nested)" in text and "second" in text and "third \\ line" in text
        assert "%PDF" not in text and "endobj" not in text and "Tj" not in text
        assert text.index("Hello") < text.index("second") < text.index("third")


# ------------------------------------------------------------------------------ hashes / determinism
def test_content_hash_is_sha256_of_the_extracted_text_not_of_the_input():
    cases = [(b"<p>Hello</p>", "html"), (HELLO_PDF, "pdf"), (rb"Text with $x$.", "latex")]
    for raw, fmt in cases:
        a, b = EX.extract(raw, fmt), EX.extract(raw, fmt)
        assert a.content_hash == hashlib.sha256(a.text.encode()).hexdigest()
        assert fmt == "latex" or a.content_hash != hashlib.sha256(raw).hexdigest()
        assert (a.text, a.content_hash, a.format, a.bytes_in) == (b.text, b.content_hash, b.format, b.bytes_in) and a.bytes_in == len(raw)
    d = EX.ExtractedDocument("abc", "html", "s", 999)
    assert d.content_hash == "ba7816bf8f01cfea414140de5dae2223b00361a396177a9cb410ff61f20015ad" and d.bytes_in == 999
    assert EX.ExtractedDocument("", "latex", None, 0).content_hash == "e3b0c44298fc1c149afbf4c8996fb92427ae41e4649b934ca495991b7852b855"
