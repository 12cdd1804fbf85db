"""Writes two small fixtures from the reference tree (run where it is mounted):

  driver_expected.json  stdout each hot-path test driver must print (test/*.output.expected)
  klas_symbols.txt      the mangled names the reference's Klas objects export
                        (from oracle/_ref/symbols.json, i.e. nm of dist/Klas_*.cu built for sm_100a)

    python oracle/build.py --ref-root /path/to/kuiper && python tests/golden/make_driver_fixtures.py /path/to/kuiper
(the path may also come from the KUIPER_REF_ROOT environment variable)
"""
import json
import os
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
REPO = HERE.parent.parent
if len(sys.argv) < 2 and not os.environ.get("KUIPER_REF_ROOT"):
    sys.exit("usage: make_driver_fixtures.py /path/to/kuiper   (or set KUIPER_REF_ROOT)")
ref_root = Path(sys.argv[1] if len(sys.argv) > 1 else os.environ["KUIPER_REF_ROOT"])

expected = {}
for pat in ("Test_Kuiper_GraphDist.output.expected", "Test_Klas_GEMM_*.output.expected", "Test_Klas_SPMM__*.output.expected",
            "Test_Klas_Softmax__*.output.expected", "Test_Klas_LogSoftmax__*.output.expected",
            "Test_Klas_HReduce__*.output.expected", "Test_Klas_AtomicReduce__*.output.expected"):
    for f in sorted((ref_root / "test").glob(pat)):
        expected[f.name[:-len(".output.expected")]] = f.read_text()
(HERE / "driver_expected.json").write_text(json.dumps(expected, indent=1, sort_keys=True))

symbols = json.loads((REPO / "oracle" / "_ref" / "symbols.json").read_text())
(HERE / "klas_symbols.txt").write_text("\n".join(sorted(symbols.values())) + "\n")
print(len(expected), "drivers,", len(symbols), "symbols")
