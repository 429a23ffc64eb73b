"""CPU oracle for the gated-delta / Mamba-3 sequence-mixing path.

TEST INFRASTRUCTURE ONLY.  Nothing in ``mixlab_b200`` imports this package.
It is a CPU restatement (torch on CPU, float64 unless asked otherwise) of the
reference algorithms, used by ``tests/``, by ``__graft_entry__.smoke()`` and by
the ``cpu_baseline`` / ``--impl reference`` legs of ``bench.py`` as the
checker and as the timed CPU baseline - never as a compute path of the
product.

Parity status: PINNED.  ``tests/golden/*.json`` hold input/output vectors
produced by running the reference's own pure-Python scalar implementations
(``experiments/gated_deltanet_reference/generate_fixtures.py``,
``experiments/mamba3_reference/generate_fixtures.py``,
``experiments/gated_deltanet_test/dump_fla_reference_pure.py``,
``train/hf_templates/mamba3_mixlab.py``) and the reference's checked-in
``train/testdata/*_full_block_reference.json`` expected outputs;
``tests/golden/make_golden.py`` is the script that produced them.
"""
