"""The public header is plain C and the shared library links from a C program (no GPU calls made):
the same boundary a Rust `extern "C"` block, cgo or JNI stub would bind."""
import os
import subprocess
import textwrap

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_header_compiles_as_c_and_library_links(tmp_path):
    import __graft_entry__ as ge
    ge.build()
    src = tmp_path / "client.c"
    src.write_text(textwrap.dedent(r"""
        #include <stdio.h>
        #include <string.h>
        #include "atenia_moe.h"
        int main(void) {
          AteniaMoeConfig cfg;
          AteniaMoeLayer* layer = NULL;
          AteniaMoeStack* stack = NULL;
          int64_t so[2], sc[2], ro[2], rc[2], tot = -1;
          int32_t counts[2 * 4] = {1, 2, 3, 4, 5, 6, 7, 8};
          memset(&cfg, 0, sizeof cfg);
          if (atenia_moe_create(NULL, &layer) != ATENIA_ERR_NULL) return 1;
          if (atenia_moe_create(&cfg, &layer) != ATENIA_ERR_SHAPE || layer != NULL) return 2;
          if (strcmp(atenia_moe_status_str(ATENIA_OK), "ok") != 0) return 3;
          if (atenia_execute_real_moe_layer(99, NULL, 0, NULL) != ATENIA_ERR_LAYER_NOT_FOUND) return 4;
          if (atenia_moe_stack_create(NULL, 0, 0, &stack) != ATENIA_ERR_NULL) return 5;
          if (atenia_moe_dispatch_noalloc(NULL, 0, 1, 1, NULL, NULL, NULL, NULL) != ATENIA_ERR_NULL) return 6;
          if (atenia_tier_detect_dtype("/nonexistent/file.bin", 1, 1) != ATENIA_ERR_IO) return 7;
          /* expert e lives on rank e / 2: rank 0 sends 1+2 to itself and 3+4 to rank 1, receives 1+2 and 5+6 */
          if (atenia_moe_ep_plan(counts, 2, 4, 0, so, sc, ro, rc, NULL, &tot) != ATENIA_OK) return 8;
          if (sc[0] != 3 || sc[1] != 7 || rc[0] != 3 || rc[1] != 11 || tot != 14 || so[1] != 3 || ro[1] != 3) return 9;
          printf("%d\n", atenia_moe_ep_unique_id_bytes());
          return 0;
        }
    """))
    exe = tmp_path / "client"
    libdir = os.path.join(ROOT, "ateniaengine_b200", "csrc")
    subprocess.check_call(["gcc", "-std=c11", "-Wall", "-Wextra", "-Werror", "-pedantic", "-I",
                           os.path.join(ROOT, "include"), str(src), "-o", str(exe), "-L", libdir, "-latenia_moe",
                           f"-Wl,-rpath,{libdir}"])
    out = subprocess.run([str(exe)], capture_output=True, text=True)
    assert out.returncode == 0, f"client exited with {out.returncode}: {out.stderr}"
    assert out.stdout.strip() == "128"
