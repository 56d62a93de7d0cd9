"""CPU checker for the attention path - TEST INFRASTRUCTURE ONLY.

Only tests/, the smoke check and the benchmark's cpu_baseline / reference arm may import this
package.  The product (granite_b200, libgranite_cuda.so) never does.
"""
