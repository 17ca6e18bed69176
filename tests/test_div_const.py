"""The scale division x / qmax is done on the device by a multiply and two FMAs; this is the exhaustive proof that
the result is the IEEE quotient for every input the kernels can see (all floats in [1e-8, 3e38], qmax 127 and 7)."""
import os
import subprocess


def test_fma_division_by_qmax_is_exact(tmp_path):
    here = os.path.dirname(os.path.abspath(__file__))
    exe = str(tmp_path / 'div_const_check')
    subprocess.run(['gcc', '-O2', '-fopenmp', '-ffp-contract=off', '-o', exe, os.path.join(here, 'div_const_check.c'), '-lm'],
                   check=True)
    r = subprocess.run([exe], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout
    assert r.stdout.count('mismatches 0') == 2, r.stdout


def test_fma_division_by_fp16_factor_is_exact(tmp_path):
    """GGA's row and column factors are fp16 values; the kernels divide by them with a multiply and two FMAs."""
    here = os.path.dirname(os.path.abspath(__file__))
    exe = str(tmp_path / 'div_h16_check')
    subprocess.run(['gcc', '-O2', '-fopenmp', '-ffp-contract=off', '-o', exe, os.path.join(here, 'div_h16_check.c'), '-lm'],
                   check=True)
    r = subprocess.run([exe], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and 'mismatches 0 ' in r.stdout, r.stdout


def test_fixed_point_pass_arithmetic(tmp_path):
    """The staged kernel's integer state pass: byte slices of the 24-bit fixed-point q / k recombine exactly, the
    int4 offset is carried by the slice sums' start values, and a chunk sum stays within the fixed-point rounding of
    the double-precision dot product."""
    here = os.path.dirname(os.path.abspath(__file__))
    exe = str(tmp_path / 'fx_pass_check')
    subprocess.run(['gcc', '-O2', '-ffp-contract=off', '-o', exe, os.path.join(here, 'fx_pass_check.c'), '-lm'], check=True)
    r = subprocess.run([exe], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and 'failures 0' in r.stdout, r.stdout
