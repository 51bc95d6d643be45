cd /root/repo/_work
./sk_E 14336 4096 1 1 | tail -1
PDL=1 ./sk_E 14336 4096 1 1 | tail -1
for M in 2 4 8 16; do PDL=1 ./sk_E 14336 4096 $M 1 | tail -1; done
for M in 1 4; do PDL=1 ./sk_E 4096 14336 $M 1 | tail -1; done
PDL=1 ./sk_E 8192 8192 1 2 | tail -1
PDL=1 ./sk_E 4096 4096 1 0 | tail -1
PDL=1 ./sk_E 57344 8192 1 1 | tail -1
./tr_E 14336 4096 1 1
