"""Extract the reference's 37 known-answer 16-element vectors into proof_kats.json.

Source: proof/nvfp4_bound_example.py:28-254 (EXAMPLES) of efsotr/nvfp4quant_test,
whose own verifier (:291-338) asserts that (a) round_E4M3(max|x|/6) has bit pattern
q0_bits and (b) the exhaustive float64 optimum over all positive finite E4M3 scales is
q0_bits + offset with a strict gap.  This script re-runs that verifier and stores the
vectors with their expected answers so the tests need no access to the reference tree.

  python tests/golden/make_proof_kats.py /path/to/reference
"""
import json
import pathlib
import sys

import numpy as np


def main() -> None:
    if len(sys.argv) < 2:
        raise SystemExit("usage: make_proof_kats.py /path/to/nvfp4quant_test")
    ref = pathlib.Path(sys.argv[1])
    sys.path.insert(0, str(ref / "proof"))
    import nvfp4_bound_example as ex  # noqa: E402

    ex.verify_examples()
    rows = []
    for (kind, part, b, offset), y in ex.EXAMPLES:
        q0_bits = ex.q0_bits_from_part_b(part, b)
        q0_value = float(ex.fp8_value_from_bits(q0_bits))
        x = q0_value * np.array(y, dtype=float)
        best_bits, best_loss, second_bits, second_loss = ex.best_scale_bits(x)
        rows.append({
            "kind": kind, "part": part, "b": b, "offset": offset, "q0_bits": q0_bits,
            "y": list(map(float, y)), "x_f64": [float(t) for t in x],
            "best_bits": int(best_bits), "second_bits": int(second_bits),
            "rel_gap": float((second_loss - best_loss) / best_loss) if best_loss > 0 else None,
        })
    out = pathlib.Path(__file__).with_name("proof_kats.json")
    out.write_text(json.dumps(rows, indent=1) + "\n")
    print(f"wrote {len(rows)} vectors to {out}")


if __name__ == "__main__":
    main()
