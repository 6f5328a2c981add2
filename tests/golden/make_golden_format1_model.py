"""Writes tests/golden/packed_model/packed_v1/: the committed source model of packed_model/src
packed in format 1 (fixed-width codes with escapes) by the reference's own packer.

    python tests/golden/make_golden_format1_model.py /path/to/the/reference/checkout

The source shard is the one make_golden.py wrote; only the reference's numpy packer is imported.
"""

import hashlib
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent


def main(reference: Path) -> None:
    sys.path.insert(0, str(reference))
    from binade.pack import pack_model

    src, out = HERE / "packed_model" / "src", HERE / "packed_model" / "packed_v1"
    out.mkdir(parents=True, exist_ok=True)
    pack_model(src, out, chunk=5000, log=lambda *_: None, version="1")
    (out / "binade_pack.json").unlink()  # holds wall time and a git commit: not reproducible
    digest = hashlib.sha256((out / "model.safetensors").read_bytes()).hexdigest()
    (HERE / "packed_model" / "SHA256_v1").write_text(f"{digest}  packed_v1/model.safetensors\n")
    print("format-1 golden shard written;", digest)


if __name__ == "__main__":
    main(Path(sys.argv[1]))
