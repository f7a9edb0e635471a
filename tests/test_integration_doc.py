"""INTEGRATION.md quotes the OCaml sources under ocaml/; every quoted block must be text of the file it names."""
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_ocaml_excerpts_are_verbatim():
    doc = open(os.path.join(ROOT, "INTEGRATION.md")).read()
    blocks = re.findall(r"```ocaml\n\(\* file: ([^ ]+) \*\)\n(.*?)\n```", doc, flags=re.S)
    assert len(blocks) >= 6
    for path, text in blocks:
        src = open(os.path.join(ROOT, path)).read()
        assert text in src, f"an excerpt attributed to {path} is not in that file"


def test_every_status_code_of_the_header_is_mapped_in_the_ocaml_error_module():
    hdr = open(os.path.join(ROOT, "include", "sb200.h")).read()
    err = open(os.path.join(ROOT, "ocaml", "sarek-b200", "B200_error.ml")).read()
    codes = dict(re.findall(r"#define (SB200_ERR_[A-Z_]+) \((-\d+)\)", hdr))
    assert len(codes) >= 11
    for name, value in codes.items():
        ml = "err_" + name[len("SB200_ERR_"):].lower()
        assert re.search(rf"let {ml} = {value}\b", err), f"{name} ({value}) has no counterpart in B200_error.ml"
        assert err.count(ml) >= 2, f"{ml} is declared but not mapped"
