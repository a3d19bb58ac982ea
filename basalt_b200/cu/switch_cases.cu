// A switch with fall-through, a default in the middle, a nested loop with `continue`, and a switch inside
// a loop whose `break` leaves only the switch.
__global__ void switch_cases(const int *in, int *out, int n) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    int v = in[i];
    int acc = 0;
    switch (v % 6) {
        case 0:
            acc = 100;
            break;
        case 1:
            acc = 10;
        case 2:            // 1 falls through into 2
            acc += 7;
            break;
        default:           // 3 and negative remainders
            acc = -1;
        case 4:            // default falls through into 4
            acc *= 3;
            break;
        case 5: {
            int t = v / 6;
            acc = t - 1;
        }
    }
    for (int k = 0; k < 4; k++) {
        switch (k) {
            case 1:
                continue;          // the loop's continue, not the switch's
            case 2:
                acc += 1000;
                break;             // leaves the switch only
            default:
                acc += k;
        }
        acc += 1;
    }
    out[i] = acc;
}
