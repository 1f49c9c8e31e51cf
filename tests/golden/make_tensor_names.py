"""Writes tests/golden/qwen35_tensor_names.json from the tensor list the reference keeps of the checkpoint it serves
(gguf-plugin/iq3s-tensor-names.json; the reference's own adapter test reads the same file,
gguf-plugin/test_gguf_rco_cpu.py:84-128).  Kept: every tensor's name, GGML type name and dimensions, compacted by
block.  Run in the build container, where the reference tree is mounted:

    python tests/golden/make_tensor_names.py /path/to/reference
"""
import json
import os
import re
import sys


def main(ref_root: str) -> None:
    doc = json.load(open(os.path.join(ref_root, "gguf-plugin", "iq3s-tensor-names.json"), encoding="utf-8"))
    top, vision, blocks = [], [], {}
    for t in doc["tensors"]:
        name, dims, typ = t["name"], t["dims"], t["type"]
        m = re.fullmatch(r"blk\.(\d+)\.(.+)", name)
        if m:
            blocks.setdefault(int(m.group(1)), []).append([m.group(2), typ, dims])
        elif name.startswith(("v.", "mm.")):
            vision.append(name)
        else:
            top.append([name, typ, dims])
    out = {"source": "gguf-plugin/iq3s-tensor-names.json", "file": doc.get("file"), "architecture": doc.get("architecture"),
           "top": top, "n_vision_and_projector": len(vision), "vision_examples": vision[:4],
           "blocks": {str(i): sorted(v) for i, v in sorted(blocks.items())}}
    here = os.path.dirname(os.path.abspath(__file__))
    with open(os.path.join(here, "qwen35_tensor_names.json"), "w", encoding="utf-8") as f:
        json.dump(out, f, separators=(",", ":"))
    print(len(doc["tensors"]), "tensors ->", os.path.getsize(os.path.join(here, "qwen35_tensor_names.json")), "bytes")


if __name__ == "__main__":
    if len(sys.argv) < 2:
        raise SystemExit("usage: make_tensor_names.py <path to a checkout of the reference repository>")
    main(sys.argv[1])
