//! Host-side tests of the facade (CPU backend, tape, reference transport); they need `libincin_host.so` and
//! `libincin_sm100.so` in `incin_b200/lib` (python -m incin_b200 build) on the loader path, and no GPU.
use incin_b200::autograd;
use incin_b200::prelude::*;

dim!(Batch, Hidden);

#[test]
fn shapes_are_checked_by_type_and_at_run_time() {
    let a: Tensor<s![2, 3]> = Tensor::from_vec(vec![1.0, 2.0, 3.0, 4.0, 5.0, 6.0], &[2, 3]).unwrap();
    let b: Tensor<s![3, 2]> = Tensor::from_vec(vec![1.0, 0.0, 0.0, 1.0, 1.0, 1.0], &[3, 2]).unwrap();
    let c = a.matmul(&b).unwrap();                      // Tensor<s![2, 2]>; s![2, 3] x s![2, 2] would not compile
    assert_eq!(c.dims(), &[2, 2]);
    assert_eq!(c.to_vec(), vec![4.0, 5.0, 10.0, 11.0]);
    // a dyn axis is checked when the tensor is built and when it meets another one
    let x: Tensor<s![dyn, 3]> = Tensor::zeros_dyn(&[5, 3]).unwrap();
    assert_eq!(x.matmul(&b).unwrap().dims(), &[5, 2]);
    assert!(Tensor::<s![dyn, 3]>::zeros_dyn(&[5, 4]).is_err());
    assert!(matches!(Tensor::<s![2, 3]>::from_vec(vec![0.0; 5], &[2, 3]), Err(ShapeError::Numel { .. })));
    let r: Tensor<s![3, dyn]> = a.clone().reshape(&[3, -1]).unwrap();
    assert_eq!(r.dims(), &[3, 2]);
    assert!(a.clone().reshape::<s![]>(&[4, -1]).is_err());
}

#[test]
fn slicing_checks_every_bound() {
    let t: Tensor<s![4, 6]> = Tensor::from_vec((0..24).map(|v| v as f32).collect(), &[4, 6]).unwrap();
    let s1 = t.slice(&idx![1..3, ..]).unwrap();
    assert_eq!(s1.dims(), &[2, 6]);
    assert_eq!(s1.as_slice()[0], 6.0);
    let s2 = t.slice(&idx![-1, 2..4]).unwrap();
    assert_eq!(s2.dims(), &[2]);
    assert_eq!(s2.to_vec(), vec![20.0, 21.0]);
    let s3 = t.slice(&idx![Idx::Ellipsis, 5]).unwrap();
    assert_eq!(s3.to_vec(), vec![5.0, 11.0, 17.0, 23.0]);
    assert!(matches!(t.slice(&idx![0..5, ..]), Err(ShapeError::OutOfBounds { axis: 0, .. })));
    assert!(matches!(t.slice(&idx![0, 0, 0]), Err(ShapeError::TooManyIndices { .. })));
}

#[test]
fn named_axes_bind_once() {
    let axes = shape_axes().bind::<Batch>(32).unwrap().bind::<Hidden>(128).unwrap();
    assert_eq!(axes.get::<Batch>(), Some(32));
    assert!(axes.bind::<Batch>(16).is_err());
}

fn shape_axes() -> incin_b200::shape::Axes {
    incin_b200::shape::Axes::new()
}

#[test]
fn oracle_ops_match_hand_computed_values() {
    let t: Tensor<s![1, 3]> = Tensor::from_vec(vec![-1.0, 0.0, 2.0], &[1, 3]).unwrap();
    assert_eq!(t.relu().to_vec(), vec![0.0, 0.0, 2.0]);
    let p = t.softmax(false).to_vec();
    assert!((p.iter().sum::<f32>() - 1.0).abs() < 1e-6 && p[2] > p[1] && p[1] > p[0]);
    let n = t.normalize(&[1.0, 1.0, 1.0], Some(&[0.0, 0.0, 0.0]), 1e-5, false).unwrap().to_vec();
    assert!(n.iter().sum::<f32>().abs() < 1e-5);
    assert!(t.normalize(&[1.0, 1.0], None, 1e-5, true).is_err());
}

#[test]
fn tape_trains_an_mlp_and_the_trainer_reports_steps() {
    let batches: Vec<Batch> = (0..4u64)
        .map(|i| {
            let x: Tensor<s![16, 8]> = Tensor::randn_dyn(&[16, 8], 100 + i).unwrap();
            let targets = x.as_slice().chunks(8).map(|row| (row[0] > 0.0) as i64).collect();
            Batch { inputs: x.to_vec(), rows: 16, features: 8, targets }
        })
        .collect();
    let plan = Trainer::plan().devices(DeviceSet::cpu()).epochs(30).build().unwrap();
    let mut model = Mlp::build((8, 16, 2), 0);
    let mut opt = AdamW::new(model.num_parameters(), 1e-2);
    let losses = Trainer::new(plan).fit(&mut model, &mut opt, &batches).unwrap();
    assert_eq!(losses.len(), 120);
    assert!(losses[119] < losses[0] * 0.6, "loss {} -> {}", losses[0], losses[119]);
    assert_eq!(opt.steps_taken(), 120);
    // a bad target is reported with the index of the step that failed
    let mut bad = batches.clone();
    bad[1].targets[0] = 7;
    let plan = Trainer::plan().epochs(1).build().unwrap();
    match Trainer::new(plan).fit(&mut model, &mut opt, &bad) {
        Err(TrainError::Step { index, .. }) => assert_eq!(index, 1),
        other => panic!("expected a step error, got {other:?}"),
    }
    // plans are validated before anything runs
    assert!(matches!(Trainer::plan().epochs(0).build(), Err(TrainError::NoEpochs)));
    let two = Trainer::plan().devices(DeviceSet::cuda(0..2).unwrap()).build().unwrap();
    assert!(matches!(Trainer::new(two).fit(&mut model, &mut opt, &batches), Err(TrainError::CollectivesUnavailable { devices: 2 })));
    autograd::reset();
}

#[test]
fn gradients_of_a_linear_layer() {
    autograd::reset();
    let x = Var::leaf(&[1.0, 2.0], 1, 2, false).unwrap();
    let w = Var::leaf(&[0.5, -0.5, 1.0, 1.0], 2, 2, true).unwrap();
    let y = x.linear(&w, None).unwrap();                 // [-0.5, 3.0]
    assert_eq!(y.value().unwrap(), vec![-0.5, 3.0]);
    let loss = y.cross_entropy(&[1]).unwrap();
    let grads = loss.backward().unwrap();
    let gw = grads.get(&w).unwrap();
    // d loss / d logits = softmax - onehot; d / dW = that (column) times x (row)
    let p0 = 1.0 / (1.0 + (3.5f32).exp());
    assert!((gw[0] - p0 * 1.0).abs() < 1e-5 && (gw[1] - p0 * 2.0).abs() < 1e-5);
    assert!((gw[2] + p0 * 1.0).abs() < 1e-5 && (gw[3] + p0 * 2.0).abs() < 1e-5);
    let gx = grads.get(&x).unwrap();                     // d / dx = dlogits W
    assert!((gx[0] + 0.5 * p0).abs() < 1e-5 && (gx[1] + 1.5 * p0).abs() < 1e-5);
    assert_eq!(autograd::depth(), 0);                    // backward drains the tape
    let v = no_grad(|| x.linear(&w, None).unwrap());
    assert_eq!(autograd::depth(), 0);
    assert_eq!(v.cols(), 2);
}

#[test]
fn reference_transport_and_mesh() {
    let t = ReferenceTransport;
    let ranks = vec![vec![1.0f32, 2.0, 3.0, 4.0], vec![10.0, 20.0, 30.0, 40.0]];
    assert_eq!(t.all_reduce(&ranks, ReduceOp::Sum).unwrap()[1], vec![11.0, 22.0, 33.0, 44.0]);
    assert_eq!(t.all_reduce(&ranks, ReduceOp::Mean).unwrap()[0], vec![5.5, 11.0, 16.5, 22.0]);
    assert_eq!(t.all_gather(&ranks).unwrap()[0].len(), 8);
    assert_eq!(t.reduce_scatter(&ranks, ReduceOp::Sum).unwrap(), vec![vec![11.0, 22.0], vec![33.0, 44.0]]);
    assert_eq!(t.all_to_all(&ranks).unwrap(), vec![vec![1.0, 2.0, 10.0, 20.0], vec![3.0, 4.0, 30.0, 40.0]]);
    assert!(t.reduce_scatter(&[vec![1.0; 3], vec![1.0; 3]], ReduceOp::Sum).is_err());

    let m = mesh![dp = 2, tp = 4];
    assert_eq!(m.size(), 8);
    assert!(m.validate(8).is_ok() && m.validate(4).is_err());
    assert_eq!(m.coordinates(5), (1, 0, 1));
    assert_eq!(Placement::Sharded(0).transition(Placement::Replicated), Some("all_gather"));
    assert_eq!(Placement::PartialSum.transition(Placement::Sharded(1)), Some("reduce_scatter(sum)"));
    assert_eq!(Placement::Replicated.transition(Placement::PartialSum), None);

    // a process started without launcher variables is a world of one
    let ctx = DistributedContext::from_env().unwrap();
    assert!(ctx.rank < ctx.world);
}

#[test]
fn safetensors_roundtrip_keeps_names_shapes_and_values() {
    let dir = std::env::temp_dir().join(format!("incin_b200_facade_{}", std::process::id()));
    std::fs::create_dir_all(&dir).unwrap();
    let path = dir.join("mlp.safetensors");
    let model = Mlp::build((8, 16, 2), 3);
    model.save(Format::Safetensors, &path).unwrap();
    let tensors = load_safetensors(&path).unwrap();
    let names: Vec<&str> = tensors.iter().map(|t| t.name.as_str()).collect();
    assert_eq!(names, vec!["0.weight", "0.bias", "2.weight", "2.bias"]);
    assert_eq!(tensors[0].shape, vec![16, 8]);
    assert_eq!(tensors[0].data, model.fc1.weight);
    let mut other = Mlp::build((8, 16, 2), 4);
    assert_ne!(other.fc2.bias, model.fc2.bias);
    other.load(&path).unwrap();
    assert_eq!(other.fc2.bias, model.fc2.bias);
    let mut wrong = Mlp::build((8, 32, 2), 0);
    assert!(wrong.load(&path).is_err());
    std::fs::remove_dir_all(&dir).unwrap();
}

#[test]
fn native_runtime_digest_loader_and_telemetry() {
    use incin_b200::runtime::{BatchLoader, Digest, TelemetrySink};
    assert_eq!(Digest::new().finish(), 0xCBF29CE484222325);
    assert_eq!(Digest::new().bytes(b"a").finish(), 0xAF63DC4C8601EC8C);      // published FNV-1a 64 vector
    assert_ne!(Digest::new().text("ab").finish(), Digest::new().text("a").text("b").finish());   // fields are length-prefixed

    let inputs: Vec<f32> = (0..40).map(|v| v as f32).collect();               // 20 rows of 2
    let targets: Vec<i64> = (0..20).collect();
    let mut seen = Vec::new();
    for workers in [1usize, 4] {
        let mut ld = BatchLoader::new(&inputs, 2, Some(&targets), 6, true, false, 3, workers, 2).unwrap();
        assert_eq!(ld.start(0), 4);
        let mut order = Vec::new();
        while let Some(b) = ld.next_batch() {
            assert_eq!(b.inputs.len(), b.rows * 2);
            for (i, t) in b.targets.iter().enumerate() {
                assert_eq!(b.inputs[2 * i], (2 * t) as f32);                   // rows of both arrays stay aligned
            }
            order.extend(b.targets);
        }
        let mut sorted = order.clone();
        sorted.sort();
        assert_eq!(sorted, targets);
        seen.push(order);
    }
    assert_eq!(seen[0], seen[1]);                                             // independent of the worker count

    let path = std::env::temp_dir().join(format!("incin_b200_telemetry_{}.jsonl", std::process::id()));
    {
        let sink = TelemetrySink::open(&path, 64).unwrap();
        assert!(sink.scalar("loss", 0.5, 1));
        assert_eq!(sink.flush(), 0);
    }
    let text = std::fs::read_to_string(&path).unwrap();
    assert!(text.contains("\"kind\":\"scalar\"") && text.contains("\"name\":\"loss\""));
    std::fs::remove_file(&path).unwrap();
}
