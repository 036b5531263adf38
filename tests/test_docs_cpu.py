"""The user documentation stays true: every flag of every app is documented where the app is described, the documents name
no flag that does not exist, and every environment variable the code reads is listed."""
import argparse
import re
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
DOCS = ROOT / "docs" / "user"


def _flags(ap: argparse.ArgumentParser):
    out = set()
    for a in ap._actions:
        if isinstance(a, argparse._SubParsersAction):
            for sp in a.choices.values():
                out |= _flags(sp)
        else:
            out |= {o for o in a.option_strings if o.startswith("--") and o != "--help"}
    return out


def _doc_flags(name: str):
    return set(re.findall(r"(?<![\w-])--[a-z][a-z0-9-]*", (DOCS / name).read_text()))


def test_every_app_flag_is_documented_and_no_documented_flag_is_missing():
    from phaseshift_b200.apps import bench, compute, gpu_test_runner, quantizer, server, tools
    for mod, doc in ((compute, "compute.md"), (server, "server.md"), (quantizer, "quantizer.md"), (bench, "bench.md"),
                     (tools, "tools.md"), (gpu_test_runner, "gpu_test_runner.md")):
        have, said = _flags(mod.build_parser()), _doc_flags(doc)
        assert have - said == set(), (doc, "undocumented", sorted(have - said))
        assert said - have == set(), (doc, "documented but absent", sorted(said - have))
    from phaseshift_b200.apps import cli
    assert _flags(cli.build_parser()) == _doc_flags("cli.md"), sorted(_flags(cli.build_parser()) ^ _doc_flags("cli.md"))


def test_every_environment_variable_read_by_the_code_is_listed():
    pat = re.compile(r"(?:environ\.get\(|environ\[|getenv\(|env\.get\()\s*[\"'](PS_[A-Z0-9_]+)[\"']")
    read = set()
    for p in list((ROOT / "phaseshift_b200").rglob("*.py")) + list((ROOT / "phaseshift_b200" / "csrc").rglob("*.cu*")) + \
            list((ROOT / "phaseshift_b200" / "csrc").rglob("*.h")) + list((ROOT / "phaseshift_b200" / "csrc").rglob("*.cpp")):
        read |= set(pat.findall(p.read_text(errors="ignore")))
    listed = set(re.findall(r"`(PS_[A-Z0-9_]+)`", (DOCS / "environment.md").read_text()))
    internal = {"PS_TP_SPAWNED"}                      # set by the launcher for the ranks it starts, not a user setting
    assert read - listed - internal == set(), sorted(read - listed - internal)
    assert {v for v in listed if v.startswith("PS_DEV_")} <= {"PS_DEV_CHECK_FAILED", "PS_DEV_WAIT_TIMEOUT"}
    stale = {v for v in listed if not v.startswith("PS_DEV_")} - read - {"PS_TEST_VRAM_GIB"}     # exported to tests, read by nobody here
    assert stale == set(), sorted(stale)
