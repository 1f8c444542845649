# Turns the `ptxas -v` report of fused_tc_kernel.cu into rows of a C table:
#   {BN, STAGES, CLUSTER, EPI, PAIR, OUT32, KD, TM, registers, spill store bytes, spill load bytes, stack bytes},
# one per instantiated variant of the kernel template (the template arguments are read off
# the mangled entry name).
/Compiling entry function/ {
  have = match($0, /fused_tc_kernelILi[0-9]+ELi[0-9]+ELb[01]ELi[0-9]+ELb[01]ELb[01]ELi[0-9]+ELi[0-9]+E/)
  if (have) {
    name = substr($0, RSTART, RLENGTH)
    n = split(name, part, /ELi|ELb|ILi|E$/)
    bn = part[2]; st = part[3]; cl = part[4]; ep = part[5]; pa = part[6]; o32 = part[7]; kd = part[8]; tm = part[9]
  }
}
/bytes stack frame/ && have {
  match($0, /[0-9]+ bytes stack frame/); stack = substr($0, RSTART, RLENGTH) + 0
  match($0, /[0-9]+ bytes spill stores/); ss = substr($0, RSTART, RLENGTH) + 0
  match($0, /[0-9]+ bytes spill loads/); sl = substr($0, RSTART, RLENGTH) + 0
}
/Used [0-9]+ registers/ && have {
  match($0, /Used [0-9]+ registers/); regs = substr($0, RSTART + 5, RLENGTH - 5) + 0
  printf("{%d, %d, %d, %d, %d, %d, %d, %d, %d, %d, %d, %d},\n", bn, st, cl, ep, pa, o32, kd, tm, regs, ss, sl, stack)
  have = 0
}
