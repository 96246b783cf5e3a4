"""Every measurement command that a file under ``profiles/`` names exists in the package."""
import re
from pathlib import Path

from kareus_b200.kernels import profile_cases

ROOT = Path(__file__).resolve().parents[1]


def test_profile_commands_name_existing_cases():
    named = set()
    for md in (ROOT / "profiles").glob("*.md"):
        named.update(re.findall(r"profile_cases\s+([a-z_0-9]+)", md.read_text()))
    assert named, "profiles/ names no measurement command"
    missing = sorted(named - set(profile_cases.CASES))
    assert not missing, f"profiles/ name cases that profile_cases does not have: {missing}"


def test_every_case_is_dispatched():
    src = Path(profile_cases.__file__).read_text()
    for case in profile_cases.CASES:
        assert f'"{case}"' in src.split("def main(")[1], case


def test_profiles_hold_text_only_and_name_no_scratch_paths():
    for p in (ROOT / "profiles").iterdir():
        assert p.suffix in (".md", ".txt"), p.name
        text = p.read_text()
        assert "_work/" not in text and "gpurun_out" not in text, p.name
