"""CPU oracle for the FP8 block-scaled GEMM. Test infrastructure only: the product
package never imports this; only tests/, __graft_entry__.smoke() and bench.py's CPU
baseline legs do."""
