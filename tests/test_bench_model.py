"""The byte model behind the bench's roofline figures, checked without a GPU: the rows of the GEMM-boundary model, taken
once per launch of a 16-bit step, add up to the whole-stack figure the stack fraction is quoted on."""
import bench


def test_model_rows_add_up_to_the_stack_figure():
    rows = sum(n * bench.boundary_model_bytes(k, 2) for k, n in bench.STEP_LAUNCHES_16BIT.items()
               if not k.startswith("readout."))
    assert rows + bench.MODEL_READOUT_BYTES == bench.MODEL_BYTES_16BIT == 37471872
    assert sum(bench.STEP_LAUNCHES_16BIT.values()) == 24          # what the engine reports as launches per classify


def test_bytes_that_cross_are_below_the_model_where_a_boundary_was_removed():
    for k in ("gdn_inproj", "gemm.sisa_in", "sisa_attn", "ffn_fused"):
        assert bench.algorithmic_work(k, 2)[0] < bench.boundary_model_bytes(k, 2)
    # the scan and the chunk preparation together against the scan's row of the model
    crossing = bench.algorithmic_work("gdn_scan", 2)[0] + bench.algorithmic_work("gdn_prep", 2)[0]
    assert crossing < bench.boundary_model_bytes("gdn_scan", 2)
    assert bench.boundary_model_bytes("gdn_prep", 2) == 0
    for k in ("assemble_norm", "rmsnorm", "gemm.o_proj"):
        assert bench.algorithmic_work(k, 2)[0] == bench.boundary_model_bytes(k, 2)
