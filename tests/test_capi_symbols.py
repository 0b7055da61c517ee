"""The launcher library loads without a GPU and exports what the header declares."""
import ctypes
import re
import subprocess

from conftest import ROOT

HEADER = ROOT / "include" / "cuda_agent_b200.h"


def declared_functions():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b([a-z][a-z0-9_]*)\s*\([^;{]*\)\s*;", text)))


def test_header_declares_the_expected_entry_points():
    names = declared_functions()
    for required in ("axpby_launcher", "gdn_decode_launcher", "cab_status_string", "cab_version"):
        assert required in names


def test_library_exports_every_declared_symbol(built_libs):
    lib = ctypes.CDLL(str(built_libs.CAPI_LIB))
    for name in declared_functions():
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"


def test_ctypes_table_covers_the_header(built_libs):
    from cuda_agent_b200 import capi
    assert sorted(capi.SIGNATURES) == declared_functions()
    assert capi.status_string(0) == "ok"
    assert capi.lib().cab_version() >= 100


def test_header_compiles_as_plain_c(tmp_path):
    src = tmp_path / "t.c"
    src.write_text('#include "cuda_agent_b200.h"\nint main(void){return CAB_OK;}\n')
    subprocess.run(["gcc", "-std=c99", "-Wall", "-Werror", "-I", str(HEADER.parent), "-c", str(src),
                    "-o", str(tmp_path / "t.o")], check=True)


def test_launchers_reject_bad_arguments_before_touching_the_device(built_libs):
    """Argument checks run on the host: callable with no GPU present."""
    from cuda_agent_b200 import capi
    lib = capi.lib()
    assert lib.axpby_launcher(None, None, None, 1.0, 0, 0, None) == 0       # size 0: no-op
    assert lib.axpby_launcher(None, None, None, 1.0, 8, 0, None) == 1       # null pointers
    assert lib.gdn_decode_launcher(None, None, None, None, None, None, None, 0, 1, 1, 0, None) == 0
    assert lib.gdn_decode_launcher(None, None, None, None, None, None, None, 2, 1, 1, 0, None) == 1
    fake = 0x1000  # aligned, never dereferenced: the shape check fails first
    assert lib.gdn_decode_launcher(fake, fake, fake, fake, fake, fake, fake, 2, 3, 4, 0, None) == 1
    assert lib.gdn_decode_launcher(fake + 4, fake, fake, fake, fake, fake, fake, 2, 2, 4, 0, None) == 2


def test_extension_registers_every_launcher_family(built_libs):
    """Every launcher family in the header (axpby_, gdn_, moe_, mla_) has ops registered."""
    import cuda_agent_b200
    ext = cuda_agent_b200.load_extension()
    ops = set(ext.registered_ops())
    families = {name.split("_")[0] for name in declared_functions() if name.endswith("_launcher")}
    for fam in families:
        assert any(op.startswith(fam) for op in ops), f"no REGISTER_BINDING for the {fam}_* launchers"
