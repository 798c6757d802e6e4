"""Renders the reference's table-batched CPU operator template into C++.

TEST INFRASTRUCTURE.  The reference keeps its CPU form of
``int_nbit_split_embedding[_nobag]_codegen_forward_{unweighted,weighted}_cpu``,
``pruned_hashmap_insert/lookup_*_cpu`` and ``pruned_array_lookup_cpu`` in a
Jinja template
(fbgemm_gpu/codegen/inference/embedding_forward_quantized_cpu_template.cpp of
FBGEMM).  This script renders it, unchanged, for ``weighted`` False and True
into the directory given; oracle/Makefile compiles the result against torch's
ATen headers.  Nothing of the reference is stored in this repository: the
output directory is a build directory.

    python oracle/render_tbe_template.py <reference root> <output dir>
"""
import os
import sys

import jinja2

TEMPLATE = "fbgemm_gpu/codegen/inference/embedding_forward_quantized_cpu_template.cpp"


def main(ref_root: str, out_dir: str) -> None:
    with open(os.path.join(ref_root, TEMPLATE)) as f:
        template = jinja2.Template(f.read(), undefined=jinja2.StrictUndefined)
    os.makedirs(out_dir, exist_ok=True)
    for weighted in (False, True):
        name = "tbe_cpu_%s.cpp" % ("weighted" if weighted else "unweighted")
        with open(os.path.join(out_dir, name), "w") as f:
            f.write(template.render(weighted=weighted))


if __name__ == "__main__":
    main(sys.argv[1], sys.argv[2])
