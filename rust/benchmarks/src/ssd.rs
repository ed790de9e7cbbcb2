//! SSD cases for the reference's benchmark binary: add `mod ssd;` to benchmarks/src/main.rs and call
//! `ssd::run_ssd_benchmarks(&mut suite, device)` beside `run_model_benchmarks` (benchmarks/src/main.rs:95-99).
//!
//! Four cases per configuration, named as the removed Mamba-2 layer's entries were
//! (benchmark_results/bench_20260112_070055.json:7,16,25,34): `ssd_forward_train`, `ssd_fwd_bwd_train`, `ssd_infer_prefill`,
//! `ssd_infer_step`.  Timing follows the binary's own convention (benchmarks/src/main.rs:140-163, 207-228): 10 warm-ups,
//! 100 iterations between device syncs, wall clock divided by the iteration count; results go into the same
//! `BenchmarkSuite` schema (benchmarks/src/results.rs:8-38).
//!
//! UNBUILT: no cargo / rustc in the image this file was written in.
use crate::results::{BenchmarkResult, BenchmarkRun, BenchmarkSuite};
use std::time::Instant;
use tch::{Cuda, Device, Kind, Tensor};

struct SsdCase {
    name: &'static str,
    batch: i64,
    seqlen: i64,
    nheads: i64,
    headdim: i64,
    dstate: i64,
    chunk: i64,
    gated: bool,
}

const TRAIN_CASES: [SsdCase; 2] = [
    SsdCase { name: "cfg1_policy_train", batch: 512, seqlen: 1024, nheads: 8, headdim: 32, dstate: 64, chunk: 128, gated: false },
    SsdCase { name: "cfg3_mamba2_130m_layer", batch: 16, seqlen: 4096, nheads: 24, headdim: 64, dstate: 128, chunk: 256, gated: true },
];

fn sync_device(device: Device) {
    if let Device::Cuda(i) = device {
        Cuda::synchronize(i as i64);
    }
}

fn time_ms<F: FnMut()>(device: Device, warmup: usize, iters: usize, mut f: F) -> f64 {
    for _ in 0..warmup {
        f();
    }
    sync_device(device);
    let start = Instant::now();
    for _ in 0..iters {
        f();
    }
    sync_device(device);
    start.elapsed().as_secs_f64() * 1000.0 / iters as f64
}

/// x ~ N(0,1); dt = softplus(0.5 N(0,1) + dt_bias) with softplus(dt_bias) log-uniform in [1e-3, 1e-1]; A = -exp(U(0, ln 16));
/// B, C ~ N(0,1)/sqrt(N); D = 1 (the value distributions of the workload definition).
struct Inputs {
    x: Tensor, dt: Tensor, a: Tensor, b: Tensor, c: Tensor, d: Tensor, z: Option<Tensor>, dy: Tensor,
}

fn make_inputs(case: &SsdCase, device: Device) -> Inputs {
    let (bn, l, h, p, n) = (case.batch, case.seqlen, case.nheads, case.headdim, case.dstate);
    let f = (Kind::Float, device);
    let bf = Kind::BFloat16;
    let u = Tensor::rand([h], f);
    let dt0 = ((1e-3f64).ln() + u * (100f64).ln()).exp();
    let dt_bias = &dt0 + (-(-&dt0).expm1()).log();
    let dt = (Tensor::randn([bn, l, h], f) * 0.5 + dt_bias).softplus();
    Inputs {
        x: Tensor::randn([bn, l, h, p], f).to_kind(bf),
        dt: dt.to_kind(bf),
        a: -(Tensor::rand([h], f) * (16f64).ln()).exp(),
        b: (Tensor::randn([bn, l, 1, n], f) / (n as f64).sqrt()).to_kind(bf),
        c: (Tensor::randn([bn, l, 1, n], f) / (n as f64).sqrt()).to_kind(bf),
        d: Tensor::ones([h], f),
        z: if case.gated { Some(Tensor::randn([bn, l, h, p], f).to_kind(bf)) } else { None },
        dy: Tensor::randn([bn, l, h, p], f).to_kind(bf),
    }
}

pub fn run_ssd_benchmarks(suite: &mut BenchmarkSuite, device: Device) {
    println!("--- SSD (Mamba-2 chunk scan) Benchmarks ---");
    let dtype = Kind::BFloat16;
    for case in TRAIN_CASES.iter() {
        let inp = make_inputs(case, device);
        let run = BenchmarkRun { batch: case.batch, seq_len: case.seqlen, dtype: format!("{:?}", dtype) };
        let z = inp.z.as_ref();
        let tokens = (case.batch * case.seqlen) as f64;

        let fwd_ms = tch::no_grad(|| {
            time_ms(device, 10, 100, || {
                let _ = ssd::forward(&inp.x, &inp.dt, &inp.a, &inp.b, &inp.c, Some(&inp.d), z, None, None, false, case.chunk, ssd::Algo::Auto)
                    .expect("ssd forward");
            })
        });
        println!("  {} forward:      {:.3} ms/iter  ({:.3e} tokens/s)", case.name, fwd_ms, tokens / (fwd_ms * 1e-3));
        suite.add(BenchmarkResult::new(&format!("ssd_forward_train_{}", case.name), fwd_ms, run.clone()));

        let fb_ms = time_ms(device, 10, 100, || {
            let out = ssd::forward(&inp.x, &inp.dt, &inp.a, &inp.b, &inp.c, Some(&inp.d), z, None, None, false, case.chunk, ssd::Algo::Auto)
                .expect("ssd forward");
            let _ = ssd::backward(&inp.dy, &inp.x, &inp.dt, &inp.a, &inp.b, &inp.c, Some(&inp.d), z, None, None, None, false, case.chunk,
                                  ssd::Algo::Auto, &out.workspace)
                .expect("ssd backward");
        });
        println!("  {} fwd+bwd:      {:.3} ms/iter  ({:.3e} tokens/s)", case.name, fb_ms, tokens / (fb_ms * 1e-3));
        suite.add(BenchmarkResult::new(&format!("ssd_fwd_bwd_train_{}", case.name), fb_ms, run.clone()));

        // prefill: the forward whose final state seeds the streamed rollout (the cached-prefill twin of
        // trading_bots/src/torch/world_model.rs:1099-1103)
        let pre_ms = tch::no_grad(|| {
            time_ms(device, 10, 100, || {
                let out = ssd::forward(&inp.x, &inp.dt, &inp.a, &inp.b, &inp.c, Some(&inp.d), z, None, None, false, case.chunk, ssd::Algo::Auto)
                    .expect("ssd prefill");
                let _ = out.final_state;
            })
        });
        println!("  {} prefill:      {:.3} ms/iter", case.name, pre_ms);
        suite.add(BenchmarkResult::new(&format!("ssd_infer_prefill_{}", case.name), pre_ms, run.clone()));
    }

    // streamed rollout: 8192 environment streams, one timestep per call, state updated in place
    let (s, h, p, n) = (8192i64, 8i64, 32i64, 64i64);
    let f = (Kind::Float, device);
    let mut state = Tensor::randn([s, h, p, n], f) * 0.1;
    let a = -(Tensor::rand([h], f) * (16f64).ln()).exp();
    let d = Tensor::ones([h], f);
    let x = Tensor::randn([s, h, p], f).to_kind(dtype);
    let dt = (Tensor::randn([s, h], f) * 0.5 - 3.0).softplus().to_kind(dtype);
    let b = (Tensor::randn([s, 1, n], f) / 8.0).to_kind(dtype);
    let c = (Tensor::randn([s, 1, n], f) / 8.0).to_kind(dtype);
    let step_ms = tch::no_grad(|| {
        time_ms(device, 10, 100, || {
            let _ = ssd::state_update(&mut state, &x, &dt, &a, &b, &c, Some(&d), None, None, false).expect("ssd step");
        })
    });
    println!("  cfg2_rollout_decode step:    {:.3} ms/iter  ({:.1} steps/s)", step_ms, 1e3 / step_ms);
    suite.add(BenchmarkResult::new("ssd_infer_step_cfg2_rollout_decode", step_ms, BenchmarkRun { batch: s, seq_len: 1, dtype: format!("{:?}", dtype) }));
    println!();
}
